"""Model and engine configuration.

ModelConfig is read from the HF-format `config.json` inside the local model directory that
GPUStack mounts and passes as {{model_path}} (gpustack/worker/backends/custom.py:91-134).
EngineConfig mirrors the subset of vLLM's CLI that GPUStack's launcher composes
(gpustack/worker/backends/vllm.py:395-507): --max-model-len, --tensor-parallel-size,
--gpu-memory-utilization, --max-num-seqs, --max-num-batched-tokens, --served-model-name.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional

SUPPORTED_ARCHS = ("LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "MixtralForCausalLM")
# designs whose config.json lists their layers one by one (LayerListConfig below)
LAYER_LIST_ARCHS = ("Vodavik", "Danipel", "Resevik", "Dotorax")


@dataclass
class ModelConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    architecture: str = "LlamaForCausalLM"
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple = ()                # every id that ends a turn (config.json list + generation_config.json)
    rope_scaling: Optional[dict] = None      # None = plain RoPE; {"rope_type": "llama3" | "linear", ...}
    quantization: Optional[str] = None       # "fp8" when config.json carries an fp8 quantization_config
    num_local_experts: int = 0               # Mixtral: experts per layer (0 = dense MLP)
    sliding_window: Optional[int] = None     # caps max_model_len (full attention == windowed below it)
    num_experts_per_tok: int = 0

    def __post_init__(self):
        ids = [int(t) for t in self.eos_token_ids]
        if self.eos_token_id is not None and int(self.eos_token_id) not in ids:
            ids.insert(0, int(self.eos_token_id))
        self.eos_token_ids = tuple(ids)
        if self.eos_token_id is None and ids:
            self.eos_token_id = ids[0]

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def kv_bytes_per_token(self, tp: int = 1) -> int:
        return 2 * self.num_hidden_layers * (self.num_key_value_heads // tp) * self.head_dim * 2

    def weight_bytes(self, tp: int = 1, quantization: Optional[str] = None) -> int:
        """bytes streamed per decode step on one rank (layers + lm_head + norms); the decoder linears
        are 1 byte/parameter under fp8, lm_head and norms stay bf16."""
        H, I = self.hidden_size, self.intermediate_size
        lin_b = 1 if (quantization or self.quantization) == "fp8" else 2
        mlp = 3 * I * H * max(1, self.num_local_experts)                      # all experts hot
        per_layer = (self.q_size + 2 * self.kv_size) * H + self.q_size * H + mlp
        router = self.num_local_experts * H * 2 * self.num_hidden_layers      # replicated, bf16
        norms = (2 * self.num_hidden_layers + 1) * H * 2                      # replicated
        return self.num_hidden_layers * per_layer // tp * lin_b + self.vocab_size * H // tp * 2 + norms + router

    @staticmethod
    def from_dict(d: dict) -> "ModelConfig":
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        arch = archs[0]
        if arch not in SUPPORTED_ARCHS:
            raise ValueError(f"unsupported architecture {arch}; supported: {SUPPORTED_ARCHS}")
        heads = d["num_attention_heads"]
        eos = d.get("eos_token_id")
        eos_all = [int(t) for t in eos] if isinstance(eos, list) else ([] if eos is None else [int(eos)])
        eos = eos_all[0] if eos_all else None
        rope = d.get("rope_theta")
        rp = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), dict) else None
        if rope is None and rp is not None:
            rope = rp.get("rope_theta")
        # legacy `rope_scaling` dict, or the transformers>=5 `rope_parameters` dict (same keys)
        sc = d.get("rope_scaling") if isinstance(d.get("rope_scaling"), dict) else rp
        rope_type = None if sc is None else sc.get("rope_type", sc.get("type"))
        scaling = None
        if rope_type not in (None, "default"):
            if rope_type == "llama3":
                scaling = {"rope_type": "llama3", "factor": float(sc["factor"]),
                           "low_freq_factor": float(sc.get("low_freq_factor", 1.0)),
                           "high_freq_factor": float(sc.get("high_freq_factor", 4.0)),
                           "original_max_position_embeddings": int(sc["original_max_position_embeddings"])}
            elif rope_type == "linear":
                scaling = {"rope_type": "linear", "factor": float(sc["factor"])}
            else:
                raise ValueError(f"rope scaling type {rope_type!r} is not supported (supported: default, llama3, linear)")
        quant = None
        qc = d.get("quantization_config")
        if isinstance(qc, dict):
            # per-tensor fp8 checkpoints with dynamic activation scales (what `--quantization fp8`
            # produces and what $VLLM/.../quantization/fp8.py:80-140 reads); anything else is refused
            method = qc.get("quant_method")
            if method != "fp8" or qc.get("activation_scheme", "dynamic") != "dynamic" or qc.get("weight_block_size"):
                raise ValueError(f"unsupported quantization_config {qc}: only quant_method=fp8, "
                                 "activation_scheme=dynamic, per-tensor weights are supported")
            quant = "fp8"
        n_exp = int(d.get("num_local_experts") or 0) if arch == "MixtralForCausalLM" else 0
        if n_exp and quant:
            raise ValueError("fp8 quantisation of mixture-of-experts models is not supported yet")
        # sliding-window attention is not implemented: a model that uses it is served with the
        # context capped at the window, where full attention is the same computation
        window = d.get("sliding_window") if d.get("use_sliding_window", True) else None
        return ModelConfig(
            quantization=quant, num_local_experts=n_exp, sliding_window=int(window) if window else None,
            num_experts_per_tok=int(d.get("num_experts_per_tok") or 0) if n_exp else 0,
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"], num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=heads, num_key_value_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or d["hidden_size"] // heads,
            rms_norm_eps=d.get("rms_norm_eps", 1e-5), rope_theta=float(rope or 10000.0),
            max_position_embeddings=d.get("max_position_embeddings", 8192),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", arch == "Qwen2ForCausalLM")),
            architecture=arch, eos_token_id=eos, bos_token_id=d.get("bos_token_id"),
            eos_token_ids=tuple(eos_all), rope_scaling=scaling)

    @staticmethod
    def from_pretrained(model_path: str):
        """The model class is chosen by config.json: a Llama-class ModelConfig, or a LayerListConfig for
        the designs in LAYER_LIST_ARCHS."""
        with open(Path(model_path) / "config.json") as f:
            d = json.load(f)
        if architecture_of(d) in LAYER_LIST_ARCHS:
            return LayerListConfig.from_dict(d)
        cfg = ModelConfig.from_dict(d)
        # chat checkpoints list their turn terminators (<|eot_id|>, ...) in generation_config.json
        gen = Path(model_path) / "generation_config.json"
        if gen.exists():
            try:
                e = json.loads(gen.read_text()).get("eos_token_id")
            except (OSError, ValueError):
                e = None
            extra = [int(t) for t in e] if isinstance(e, list) else ([] if e is None else [int(e)])
            cfg.eos_token_ids = tuple(dict.fromkeys(list(cfg.eos_token_ids) + extra))
            if cfg.eos_token_id is None and cfg.eos_token_ids:
                cfg.eos_token_id = cfg.eos_token_ids[0]
        return cfg

    def rope_inv_freq(self):
        """Inverse RoPE frequencies [head_dim/2] (fp32 torch tensor), with the checkpoint's frequency
        scaling applied ($VLLM/model_executor/layers/rotary_embedding/llama3_rope.py,
        linear_scaling_rope.py; same arithmetic as transformers' ROPE_INIT_FUNCTIONS)."""
        import math

        import torch

        D = self.head_dim
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float) / D))
        sc = self.rope_scaling
        if not sc:
            return inv
        if sc["rope_type"] == "linear":
            return inv / sc["factor"]
        factor, lo, hi = sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"]
        old = sc["original_max_position_embeddings"]
        low_wl, high_wl = old / lo, old / hi
        wl = 2 * math.pi / inv
        scaled = torch.where(wl > low_wl, inv / factor, inv)
        smooth = (old / wl - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wl >= high_wl) & (wl <= low_wl)
        return torch.where(is_mid, mid, scaled)

    def to_hf_dict(self) -> dict:
        extra = {"quantization_config": {"quant_method": "fp8", "activation_scheme": "dynamic"}} \
            if self.quantization == "fp8" else {}
        if self.num_local_experts:
            extra.update({"num_local_experts": self.num_local_experts, "num_experts_per_tok": self.num_experts_per_tok,
                          "sliding_window": None})
        model_type = {"MixtralForCausalLM": "mixtral", "Qwen2ForCausalLM": "qwen2", "MistralForCausalLM": "mistral"} \
            .get(self.architecture, "llama")
        return {
            **extra,
            "architectures": [self.architecture], "model_type": model_type, "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "attention_bias": self.attention_bias,
            "hidden_act": "silu", "torch_dtype": "bfloat16", "bos_token_id": self.bos_token_id or 1,
            "eos_token_id": (list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else
                             (self.eos_token_id if self.eos_token_id is not None else 2)),
            **({"rope_scaling": dict(self.rope_scaling)} if self.rope_scaling else {}),
        }


def architecture_of(d: dict) -> str:
    """`architectures: [name]` (HF) or `architecture: name`."""
    if isinstance(d.get("architecture"), str):
        return d["architecture"]
    archs = d.get("architectures") or ["LlamaForCausalLM"]
    return archs[0]


# ------------------------------------------------------------------------------ layer-list designs
@dataclass
class AttentionSpec:
    """Softmax attention mixer of a layer-list design.  Every option is a parameter, so another design can
    combine them differently: separate key / value widths, per-head RMS norm of q and k, a query
    temperature 1 + coef * ln(floor((p + 1) / every) + 1), a learned softmax sink, a sigmoid output
    gate, q/k/v biases, keys and values taken from an earlier layer's cache (kv_from), rotary positions,
    a weightless q/k norm after the rotation, a sliding window, values that are the unrotated keys."""
    heads: int
    kv_heads: int
    dim: int                       # query / key width per head
    vdim: int                      # value width per head
    scale: float
    qk_norm: bool = True
    qkv_bias: bool = True
    sink: bool = True
    gate: bool = True
    q_temp_coef: float = 0.0
    q_temp_every: int = 0          # 0 = no temperature
    kv_from: Optional[int] = None  # layer index whose cache this mixer reads
    rot: Optional["RotarySpec"] = None   # rotary positions on q and k (before the unit norm), None = no rotation
    qk_unit_norm: bool = False     # q and k over their root mean square per head AFTER the rotation, no weight
    window: int = 0                # > 0: position i sees j with 0 <= i - j < window
    values_are_keys: bool = False  # no value projection: v = k as projected (before rotation and norm); vdim == dim
    gate_per_head: bool = False    # the output gate is ONE number per head (gate projection [heads, width])
    head_temp: bool = False        # a learned factor per head on the score (tensor `temp` [heads])
    # pool > 0 (with a window): beside the window's tokens, position i sees one (mean key, mean value) per block
    # [b pool, (b + 1) pool) that lies wholly before the window, (b + 1) pool - 1 <= i - window, in the same softmax
    pool: int = 0

    kind = "attention"

    @property
    def q_width(self) -> int:
        return self.heads * self.dim

    @property
    def tile_sized(self) -> bool:
        """Keys and values share one width that is a tensor-core tile (64 / 128) and the group fits the decode
        kernel: the Llama-class attention kernels (with sink and gate) can serve this mixer in bf16."""
        return self.tokens_tile_sized and not self.pool

    @property
    def tokens_tile_sized(self) -> bool:
        """tile_sized without regard to pooled blocks: the tensor-core kernels can attend this mixer's TOKENS and hand
        over every row's log-sum-exp; the pooled blocks then continue that softmax in the generic kernel."""
        return self.dim == self.vdim and self.dim in (64, 128) and self.heads // self.kv_heads <= 16

    @property
    def gate_width(self) -> int:
        """Rows of the gate projection."""
        return 0 if not self.gate else (self.heads if self.gate_per_head else self.out_width)

    @property
    def pool_per_page(self):
        """(pooled entries a KV page can own) as a function of the page size: entry b lives in the page of its
        FIRST token, so a page of n tokens owns at most ceil(n / pool) entries."""
        return lambda page: -(-page // self.pool) if self.pool else 0

    @property
    def out_width(self) -> int:
        return self.heads * self.vdim


@dataclass
class MLSTMSpec:
    """Matrix-memory recurrent mixer (mLSTM): per-head state dim x vdim, gates capped by tanh."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    kind = "mlstm"

    @property
    def out_width(self) -> int:
        return self.heads * self.vdim


@dataclass
class LinearAttentionSpec:
    """Linear attention with a fixed decay per head and no softmax or denominator: per head a state S (dim x vdim,
    fp32, zero before a sequence's first token), S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  Options:
    a feature map on q, k and v ("silu" or None), rotary positions on q and k, a factor on k (after the rotation),
    the output norm ("all_heads": one RMS norm with a weight over the concatenated heads; "per_head": every head
    over its own root mean square, no weight) and the output gate's activation ("sigmoid" | "silu")."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    feature: Optional[str] = None
    rot: Optional["RotarySpec"] = None
    k_scale: float = 1.0
    out_norm: str = "per_head"
    gate_act: str = "sigmoid"
    type_name: str = "linear_attention"

    kind = "linear_attention"

    @property
    def out_width(self) -> int:
        return self.heads * self.vdim

    @property
    def proj_rows(self) -> int:
        """Rows of the fused projection [q | k | v | gate]."""
        return 2 * self.heads * self.dim + 2 * self.out_width


@dataclass
class GatedRecurrenceSpec:
    """Gated diagonal linear recurrence (a real-gated linear recurrent unit) with a short convolution in front.  Two
    branches of `width` channels read the mixer input: y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x) (causal,
    per channel, `conv` taps, with a bias).  The channels are cut into `blocks` equal parts with one square matrix per
    part and gate: r = sigmoid(A u + a), i = sigmoid(B u + b); decay = exp(-gate_c r softplus(lam));
    S_t = decay S_(t-1) + sqrt(1 - decay^2) i u, S = 0 before the first token; output W_o (S * y)."""
    width: int
    blocks: int
    conv: int                      # taps of the convolution (the last one multiplies the current token)
    gate_c: float = 8.0

    kind = "gated_recurrence"

    @property
    def out_width(self) -> int:
        return self.width

    @property
    def proj_rows(self) -> int:
        """Rows of the projection [y | x]."""
        return 2 * self.width


@dataclass
class SideBySideSpec:
    """Two mixers that read the same input; the mixer's output is left_scale * left + right_scale * right."""
    left: "AttentionSpec"
    right: GatedRecurrenceSpec
    left_scale: float
    right_scale: float

    kind = "side_by_side"

    @property
    def out_width(self) -> int:
        return self.left.out_width + self.right.out_width


@dataclass
class GatedLinearAttentionSpec:
    """Linear attention whose state rows decay at a data-dependent rate per key channel: per head
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q scaled by dim^(-1/2) and
    alpha = sigmoid(z)^(1/tau), z = A2 (A1 h) + b (a low-rank projection; its rank is the checkpoint's, decay_rank is
    what a randomly initialised model gets).  Every head's output is RMS-normed with one weight vector of vdim
    entries shared by the heads, multiplied by silu(G h) and projected."""
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int = 16

    kind = "gated_linear_attention"

    @property
    def out_width(self) -> int:
        return self.heads * self.vdim

    @property
    def proj_rows(self) -> int:
        """Rows of the fused projection [q | k | v | gate | decay latent]."""
        return 2 * self.heads * self.dim + 2 * self.out_width + self.decay_rank


@dataclass
class RotarySpec:
    """Rotary position encoding of the first `dims` entries of a vector.  layout "interleaved" pairs entry 2i
    with 2i+1, "half" pairs i with i + dims/2; frequencies base^(-2i/dims).  YaRN scaling (yarn_factor > 0):
    with dim(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos / sin are multiplied by 0.1 ln(factor) + 1."""
    dims: int
    base: float
    layout: str = "interleaved"
    yarn_factor: float = 0.0       # 0 = plain frequencies
    yarn_original: float = 0.0
    yarn_fast: float = 0.0
    yarn_slow: float = 0.0

    def frequencies(self):
        """(fp64 list of dims/2 angular frequencies, the factor on cos and sin)."""
        import math

        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        if self.yarn_factor <= 0.0:
            return f, 1.0

        def turn_dim(t):
            return self.dims * math.log(self.yarn_original / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))

        lo = max(math.floor(turn_dim(self.yarn_fast)), 0)
        hi = min(math.ceil(turn_dim(self.yarn_slow)), self.dims - 1)
        out = []
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f[i] / self.yarn_factor * ramp + f[i] * (1.0 - ramp))
        return out, 0.1 * math.log(self.yarn_factor) + 1.0

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.yarn_factor > 0.0:
            d["scaling"] = {"factor": self.yarn_factor, "original": self.yarn_original, "fast": self.yarn_fast,
                            "slow": self.yarn_slow}
        return d


@dataclass
class LatentAttentionSpec:
    """Attention whose keys and values are expanded from one latent per token: the cache holds, per token
    and layer, the RMS-normed latent c (kv_rank wide) and ONE rotated key part (rot_dim wide) shared by
    all heads.  Per head: key = [W_uk c | rotated part], value = W_uv c, query = [dim unrotated | rot_dim
    rotated]; q_rank > 0: queries go through their own RMS-normed latent.  sink: a learned per-head
    term exp(sink_h) in the softmax denominator."""
    heads: int
    dim: int                       # unrotated query / key width per head
    rot_dim: int                   # rotated query / key width per head (one shared key part)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotarySpec = None
    q_rank: int = 0                # 0 = queries straight from the mixer input
    sink: bool = False
    type_name: str = "latent_attention"

    kind = "latent_attention"

    @property
    def q_width(self) -> int:
        return self.heads * (self.dim + self.rot_dim)

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim

    @property
    def out_width(self) -> int:
        return self.heads * self.vdim

    @property
    def proj_rows(self) -> int:
        """Rows of the fused projection that reads the mixer input: [q or the query latent | latent + key part]."""
        return (self.q_rank if self.q_rank else self.q_width) + self.cache_width


@dataclass
class MoESpec:
    """Routed feed-forward: softmax over experts + identity router outputs; the `top` largest of score +
    correction are chosen, weighted by score / (sum of the chosen scores + 1e-20) * scale.  The last `identity`
    router outputs return the input itself.  An expert is  down(g sigmoid(1.702 g) (u + 1))  with
    g = min(gate x, limit), u = clamp(up x, -limit, limit); a shared expert of the same form (shared_ff > 0)
    runs for every token."""
    experts: int
    top: int
    ff: int
    limit: float
    identity: int = 0
    scale: float = 1.0
    shared_ff: int = 0
    shared_limit: float = 0.0
    # other routed designs: score "sigmoid" = sigmoid(z) per output instead of the softmax; renormalize False = the
    # chosen scores are the weights as they are; weight_on "input" = an expert runs on weight * x (its output is not
    # scaled again); act = the experts' gate activation ("clamped_swish" above | "silu": down(silu(gate x) * up x))
    score: str = "softmax"
    renormalize: bool = True
    weight_on: str = "output"
    act: str = "clamped_swish"


@dataclass
class MLPSpec:
    kind: str                      # "dense" | "moe"
    ff: int                        # dense: hidden width; moe: the widest hidden width (expert or shared)
    act: str = "relu2"             # dense: "relu2" = down(relu(up x)^2); "gelu_tanh" = down(gelu(gate x) * up x);
    #                                "clamped_swish" = down(g sigmoid(1.702 g) (u + 1)), g = min(gate x, limit),
    #                                u = clamp(up x, -limit, limit)
    moe: Optional[MoESpec] = None
    limit: float = 0.0


@dataclass
class LayerSpec:
    mixer: object                  # AttentionSpec | MLSTMSpec
    mlp: Optional[MLPSpec]


@dataclass
class LayerListConfig:
    """A decoder described layer by layer (config.json `layers`): each entry names its mixer, the mixer's
    sizes and its feed-forward.  The residual stream is normalised AFTER each sum:
    x <- LN(alpha * x + sublayer(x)), bias-free layer norm."""
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: list
    norm_eps: float = 1e-5
    postln_alpha: float = 1.0
    logit_scale: float = 1.0
    # residual scheme: "post_ln" (x <- LN(alpha x + f(x))) or "streams" (pre-norm; `streams` parallel copies of
    # the residual joined by learned scalars: u = sum_s in[s] x_s, y = f(norm(u)),
    # x_t <- sum_s mix[s, t] x_s + residual_mult * out[t] * y; streams == 0: one stream, x <- x + residual_mult * y)
    # "parallel": pre-norm with ONE norm per layer whose output feeds the mixer and the feed-forward side by side,
    # x <- x + mixer(norm(x)) + ff(norm(x))
    # "sandwich": a norm before and after every sublayer, x <- x + residual_mult * norm_b(f(norm_a(x)))
    residual: str = "post_ln"
    # "layernorm" (bias-free) | "tanh": tanh(alpha x) w + b, no statistics | "rms" | "rms_zero_centred": an RMS norm
    # whose stored weight is the deviation from one, x / rms(x) * (1 + w)
    norm: str = "layernorm"
    # input convolution: every sublayer reads h + conv(h) instead of its normed input h -- a causal convolution over
    # time with canon_taps taps per channel (the last tap multiplies the current token); 0 = none.  The last
    # canon_taps - 1 inputs of every sublayer are part of a sequence's state.
    canon_taps: int = 0
    learned_positions: bool = False            # x_0 = embed[token] + pos[position] (table of max_position_embeddings rows)
    # layers loop_start .. loop_stop-1 run loop_times times in a row with the same weights (every pass with its own
    # cache / state); before each pass but the first the embedding output is added to the residual
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    streams: int = 0
    residual_mult: float = 1.0
    embed_scale: float = 1.0
    max_position_embeddings: int = 1 << 20     # the design has no learned or tabulated positions
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple = ()
    # what the engine asks of any model config
    quantization: Optional[str] = None
    num_local_experts: int = 0
    sliding_window: Optional[int] = None
    tie_word_embeddings: bool = False

    family = "layer_list"

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def runs(self) -> list:
        """The order in which the layers run: [(layer index, True when the embedding output is added to the
        residual right before it)].  Caches and recurrent state belong to a RUN, weights to a layer."""
        a, b = self.loop_start, self.loop_stop
        if self.loop_times == 1 or b <= a:
            return [(l, False) for l in range(len(self.layers))]
        out = [(l, False) for l in range(a)]
        for p in range(self.loop_times):
            out += [(l, p > 0 and l == a) for l in range(a, b)]
        return out + [(l, False) for l in range(b, len(self.layers))]

    @property
    def has_state(self) -> bool:
        """True when some mixer carries a recurrent state per sequence (needs a state slot; no prefix reuse)."""
        return self.canon_taps > 1 or any(l.mixer.kind in ("mlstm", "linear_attention", "side_by_side",
                                                           "gated_linear_attention") for l in self.layers)

    def kv_owner(self, l: int) -> Optional[int]:
        """Layer whose K/V cache layer l's attention reads (itself unless kv_from), None for other mixers."""
        m = self.layers[l].mixer
        if m.kind == "side_by_side":
            return l
        if m.kind != "attention":
            return None
        return l if m.kv_from is None else int(m.kv_from)

    @property
    def n_streams(self) -> int:
        """Copies of the residual stream the runner keeps (1 unless the design has hyper-connections)."""
        return max(1, self.streams)

    def kv_bytes_per_token(self, tp: int = 1, elem_bytes: int = 2) -> int:
        mixers = [self.layers[l].mixer for l, _ in self.runs()]
        mixers = [m.left if m.kind == "side_by_side" else m for m in mixers]
        n = sum(m.kv_heads * (m.dim + m.vdim) * elem_bytes for m in mixers if m.kind == "attention" and m.kv_from is None)
        # pooled block means (fp32): ceil(16 / pool) entries per 16-token page
        n += sum(m.kv_heads * (m.dim + m.vdim) * 4 * m.pool_per_page(16) // 16 for m in mixers
                 if m.kind == "attention" and m.pool)
        return n + sum(m.cache_width * elem_bytes for m in mixers if m.kind == "latent_attention")

    def state_bytes_per_seq(self) -> int:
        n = 0
        for m in (self.layers[l].mixer for l, _ in self.runs()):
            if m.kind == "mlstm":
                z = (m.vdim + 31) // 32
                n += 4 * m.heads * (m.dim * m.vdim + z * m.dim + z)
            elif m.kind in ("linear_attention", "gated_linear_attention"):
                n += 4 * m.heads * m.dim * m.vdim
            elif m.kind == "side_by_side":
                n += 4 * m.right.width * m.right.conv          # the recurrence and its convolution's last inputs
        if self.canon_taps > 1:
            n += 4 * self.hidden_size * (self.canon_taps - 1) * sum(1 + (self.layers[l].mlp is not None) for l, _ in self.runs())
        return n

    def weight_bytes(self, tp: int = 1, quantization: Optional[str] = None) -> int:
        D, n = self.hidden_size, 0
        for l in self.layers:
            m = l.mixer
            if m.kind == "side_by_side":
                a, r = m.left, m.right
                n += D * (a.q_width + a.kv_heads * (a.dim + a.vdim)) + a.out_width * D
                n += 3 * D * r.width + 2 * r.width * r.width // r.blocks
            elif m.kind == "gated_linear_attention":
                n += D * m.proj_rows + m.decay_rank * m.heads * m.dim + m.out_width * D
            elif m.kind == "attention":
                kv = 0 if m.kv_from is not None else m.kv_heads * (m.dim + (0 if m.values_are_keys else m.vdim))
                n += D * (m.q_width + kv + m.gate_width) + m.out_width * D
            elif m.kind == "linear_attention":
                n += D * m.proj_rows + m.out_width * D
            elif m.kind == "latent_attention":
                n += D * m.proj_rows + (m.q_rank * m.q_width if m.q_rank else 0) \
                    + m.kv_rank * m.heads * (m.dim + m.vdim) + m.out_width * D
            else:
                n += D * (2 * m.heads * m.dim + 2 * m.out_width + 2 * m.heads) + m.out_width * D
            if l.mlp is not None and l.mlp.kind == "moe":
                e = l.mlp.moe
                n += 3 * D * (e.experts * e.ff + e.shared_ff) + (e.experts + e.identity) * D
            elif l.mlp is not None:
                n += (2 if l.mlp.act == "relu2" else 3) * D * l.mlp.ff
        return 2 * (n + self.vocab_size * D)

    @staticmethod
    def from_dict(d: dict) -> "LayerListConfig":
        arch = architecture_of(d)
        if arch not in LAYER_LIST_ARCHS:
            raise ValueError(f"unsupported architecture {arch}; layer-list designs: {LAYER_LIST_ARCHS}")
        if arch == "Danipel":
            return _danipel_from_dict(d)
        if arch == "Resevik":
            return _resevik_from_dict(d)
        if arch == "Dotorax":
            return _dotorax_from_dict(d)
        layers = []
        for i, e in enumerate(d["layers"]):
            mx = e["mixer"]
            if e["type"] == "attention":
                qt = mx.get("q_temp") or {}
                src = mx.get("kv_from")
                spec = AttentionSpec(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])),
                                     dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                                     scale=float(mx["scale"]), q_temp_coef=float(qt.get("coef", 0.0)),
                                     q_temp_every=int(qt.get("every", 0)), kv_from=None if src is None else int(src))
                if spec.heads % spec.kv_heads:
                    raise ValueError(f"layer {i}: heads {spec.heads} not a multiple of kv_heads {spec.kv_heads}")
                if spec.kv_from is not None:
                    if not (0 <= spec.kv_from < i) or d["layers"][spec.kv_from]["type"] != "attention" \
                            or d["layers"][spec.kv_from]["mixer"].get("kv_from") is not None:
                        raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with its own cache")
            elif e["type"] == "mlstm":
                spec = MLSTMSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                                 gate_cap=float(mx["gate_cap"]))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {e['type']!r}")
            mlp = e.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
                mlp = MLPSpec(kind="dense", ff=int(mlp["ff"]))
            layers.append(LayerSpec(mixer=spec, mlp=mlp))
        eos = d.get("eos_token_id")
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        return LayerListConfig(architecture=arch, vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                               norm_eps=float(d["norm"]["eps"]), postln_alpha=float(d.get("postln_alpha", 1.0)),
                               logit_scale=float(d.get("logit_scale", 1.0)), eos_token_ids=eos_all,
                               eos_token_id=eos_all[0] if eos_all else None, bos_token_id=d.get("bos_token_id"))

    def to_dict(self) -> dict:
        """config.json of this model (the inverse of from_dict)."""
        if self.architecture == "Danipel":
            return _danipel_to_dict(self)
        if self.architecture == "Resevik":
            return _resevik_to_dict(self)
        if self.architecture == "Dotorax":
            return _dotorax_to_dict(self)
        out = []
        for l in self.layers:
            m = l.mixer
            if m.kind == "attention":
                mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.q_temp_every:
                    mx["q_temp"] = {"coef": m.q_temp_coef, "every": m.q_temp_every}
                if m.kv_from is not None:
                    mx["kv_from"] = m.kv_from
            else:
                mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            out.append({"type": m.kind, "mixer": mx,
                        "mlp": None if l.mlp is None else {"kind": l.mlp.kind, "ff": l.mlp.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "layers": out,
                "norm": {"eps": self.norm_eps}, "postln_alpha": self.postln_alpha, "logit_scale": self.logit_scale}


def _eos_of(d: dict):
    eos = d.get("eos_token_id")
    return tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))


def _danipel_from_dict(d: dict) -> "LayerListConfig":
    """Danipel: pre-norm layers over `streams` residual copies, tanh norm, latent attention mixers
    ("latent_attention": direct queries, interleaved rotation, optional YaRN, softmax sink;
    "latent_attention_2": latent queries, half-split rotation, plain softmax), dense gated-GELU or routed
    feed-forward."""
    layers = []
    for i, e in enumerate(d["layers"]):
        mx, kind = e["mixer"], e["type"]
        if kind not in ("latent_attention", "latent_attention_2"):
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        two = kind == "latent_attention_2"
        r = mx["rot"]
        sc = r.get("scaling") or {}
        rot = RotarySpec(dims=int(r["dims"]), base=float(r["base"]), layout="half" if two else "interleaved",
                         yarn_factor=float(sc.get("factor", 0.0)), yarn_original=float(sc.get("original", 0.0)),
                         yarn_fast=float(sc.get("fast", 0.0)), yarn_slow=float(sc.get("slow", 0.0)))
        spec = LatentAttentionSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]),
                                   vdim=int(mx["vdim"]), kv_rank=int(mx["kv_rank"]), scale=float(mx["scale"]), rot=rot,
                                   q_rank=int(mx["q_rank"]) if two else 0, sink=not two, type_name=kind)
        if rot.dims % 2 or rot.dims > spec.rot_dim or rot.dims <= 0:
            raise ValueError(f"layer {i}: rot.dims {rot.dims} must be even and at most rot_dim {spec.rot_dim}")
        mlp = e.get("mlp")
        if mlp is not None:
            if mlp.get("kind") == "dense":
                mlp = MLPSpec(kind="dense", ff=int(mlp["ff"]), act="gelu_tanh")
            elif mlp.get("kind") == "moe":
                ro, ex, sh = mlp["router"], mlp["expert"], mlp.get("shared") or None
                moe = MoESpec(experts=int(ro["experts"]), top=int(ro["top"]), ff=int(ex["ff"]), limit=float(ex["limit"]),
                              identity=int(ro.get("identity") or 0), scale=float(ro.get("scale", 1.0)),
                              shared_ff=int(sh["ff"]) if sh else 0, shared_limit=float(sh["limit"]) if sh else 0.0)
                if not 1 <= moe.top <= moe.experts + moe.identity:
                    raise ValueError(f"layer {i}: top {moe.top} of {moe.experts + moe.identity} router outputs")
                mlp = MLPSpec(kind="moe", ff=max(moe.ff, moe.shared_ff), act="clamped_swish", moe=moe)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(mixer=spec, mlp=mlp))
    eos_all = _eos_of(d)
    return LayerListConfig(architecture="Danipel", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                           norm_eps=float(d["norm"]["eps"]), residual="streams", norm="tanh",
                           streams=int(d.get("streams") or 0), residual_mult=float(d.get("residual_mult", 1.0)),
                           embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), eos_token_ids=eos_all,
                           eos_token_id=eos_all[0] if eos_all else None, bos_token_id=d.get("bos_token_id"))


def _danipel_to_dict(c: "LayerListConfig") -> dict:
    out = []
    for l in c.layers:
        m = l.mixer
        mx = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
              "scale": m.scale, "rot": m.rot.to_dict()}
        if m.q_rank:
            mx["q_rank"] = m.q_rank
        mlp = None
        if l.mlp is not None and l.mlp.kind == "dense":
            mlp = {"kind": "dense", "ff": l.mlp.ff}
        elif l.mlp is not None:
            e = l.mlp.moe
            mlp = {"kind": "moe", "expert": {"ff": e.ff, "limit": e.limit},
                   "router": {"experts": e.experts, "identity": e.identity, "scale": e.scale, "top": e.top}}
            if e.shared_ff:
                mlp["shared"] = {"ff": e.shared_ff, "limit": e.shared_limit}
        out.append({"type": m.type_name, "mixer": mx, "mlp": mlp})
    d = {"architecture": "Danipel", "vocab": c.vocab_size, "width": c.hidden_size, "layers": out,
         "norm": {"eps": c.norm_eps}, "residual_mult": c.residual_mult, "embedding": {"scale": c.embed_scale}}
    if c.streams:
        d["streams"] = c.streams
    return d


def _resevik_from_dict(d: dict) -> "LayerListConfig":
    """Resevik: pre-norm layers whose ONE RMS norm feeds mixer and feed-forward side by side; mixers "lightning"
    (decayed linear attention, SiLU feature map, all heads normed together with a weight, sigmoid gate), "retention"
    (decayed linear attention, half-split rotation, k / sqrt(dim), every head over its own root mean square, SiLU gate)
    and "attention" (grouped softmax attention in a sliding window; interleaved rotation, then a weightless RMS
    norm of q and k; the values are the unrotated keys); a routed feed-forward whose sigmoid scores multiply the
    chosen experts' input; a span of layers run `times` times in a row."""
    layers = []
    for i, e in enumerate(d["layers"]):
        mx, kind = e["mixer"], e["type"]

        def rotary(layout):
            r = mx["rot"]
            rot = RotarySpec(dims=int(r["dims"]), base=float(r["base"]), layout=layout)
            if rot.dims % 2 or rot.dims <= 0 or rot.dims > int(mx["dim"]):
                raise ValueError(f"layer {i}: rot.dims {rot.dims} must be even and at most dim {mx['dim']}")
            return rot

        if kind == "attention":
            spec = AttentionSpec(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                                 vdim=int(mx.get("vdim", mx["dim"])), scale=float(mx["scale"]), qk_norm=False,
                                 qkv_bias=False, sink=False, gate=False, rot=rotary("interleaved"), qk_unit_norm=True,
                                 window=int(mx["mask"]["size"]), values_are_keys=True)
            if spec.heads % spec.kv_heads:
                raise ValueError(f"layer {i}: heads {spec.heads} not a multiple of kv_heads {spec.kv_heads}")
            if spec.vdim != spec.dim:
                raise ValueError(f"layer {i}: the values are the keys, so vdim {spec.vdim} must equal dim {spec.dim}")
            if spec.window < 1:
                raise ValueError(f"layer {i}: mask.size {spec.window} must be at least 1")
        elif kind in ("lightning", "retention"):
            decay = tuple(float(x) for x in mx["decay"])
            if len(decay) != int(mx["heads"]):
                raise ValueError(f"layer {i}: {len(decay)} decays for {mx['heads']} heads")
            ret = kind == "retention"
            spec = LinearAttentionSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                                       decay=decay, feature=None if ret else "silu", rot=rotary("half") if ret else None,
                                       k_scale=int(mx["dim"]) ** -0.5 if ret else 1.0,
                                       out_norm="per_head" if ret else "all_heads", gate_act="silu" if ret else "sigmoid",
                                       type_name=kind)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = e.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            ro, ex = mlp["router"], mlp["expert"]
            moe = MoESpec(experts=int(ro["experts"]), top=int(ro["top"]), ff=int(ex["ff"]), limit=0.0, score="sigmoid",
                          renormalize=False, weight_on="input", act="silu")
            if not 1 <= moe.top <= moe.experts:
                raise ValueError(f"layer {i}: top {moe.top} of {moe.experts} experts")
            mlp = MLPSpec(kind="moe", ff=moe.ff, act="silu", moe=moe)
        layers.append(LayerSpec(mixer=spec, mlp=mlp))
    lp = d.get("loop") or {}
    a, b, times = int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1))
    if times < 1 or not (0 <= a <= b <= len(layers)):
        raise ValueError(f"loop {lp}: needs 0 <= start <= stop <= {len(layers)} and times >= 1")
    eos_all = _eos_of(d)
    return LayerListConfig(architecture="Resevik", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                           norm_eps=float(d["norm"]["eps"]), residual="parallel", norm="rms",
                           embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), loop_start=a, loop_stop=b,
                           loop_times=times, eos_token_ids=eos_all, eos_token_id=eos_all[0] if eos_all else None,
                           bos_token_id=d.get("bos_token_id"))


def _resevik_to_dict(c: "LayerListConfig") -> dict:
    out = []
    for l in c.layers:
        m = l.mixer
        if m.kind == "attention":
            mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                  "mask": {"size": m.window}, "rot": m.rot.to_dict()}
            kind = "attention"
        else:
            mx = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            if m.rot is not None:
                mx["rot"] = m.rot.to_dict()
            kind = m.type_name
        mlp = None
        if l.mlp is not None:
            e = l.mlp.moe
            mlp = {"kind": "moe", "expert": {"ff": e.ff}, "router": {"experts": e.experts, "top": e.top}}
        out.append({"type": kind, "mixer": mx, "mlp": mlp})
    return {"architecture": "Resevik", "vocab": c.vocab_size, "width": c.hidden_size, "layers": out,
            "norm": {"eps": c.norm_eps}, "embedding": {"scale": c.embed_scale},
            "loop": {"start": c.loop_start, "stop": c.loop_stop, "times": c.loop_times}}


def _dotorax_from_dict(d: dict) -> "LayerListConfig":
    """Dotorax: learned positions added to the embedding; a zero-centred RMS norm before and after every sublayer,
    x <- x + residual_mult * norm_b(f(norm_a(x))); every sublayer reads its normed input plus a short causal
    convolution of it; mixers "attention" (grouped softmax attention, half-split rotation, one sigmoid gate per head,
    optionally on an earlier layer's keys and values), "parallel" (left: sliding-window attention with pooled blocks,
    interleaved rotation, weightless q / k norm, a temperature per head; right: a gated diagonal recurrence) and "gla"
    (gated linear attention); a clamped gated feed-forward."""
    layers = []
    raw = d["layers"]

    def attention(i, mx, layout, **kw):
        r = mx["rot"]
        rot = RotarySpec(dims=int(r["dims"]), base=float(r["base"]), layout=layout)
        if rot.dims % 2 or rot.dims <= 0 or rot.dims > int(mx["dim"]):
            raise ValueError(f"layer {i}: rot.dims {rot.dims} must be even and at most dim {mx['dim']}")
        spec = AttentionSpec(heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                             vdim=int(mx.get("vdim", mx["dim"])), scale=float(mx["scale"]), qk_norm=False, qkv_bias=False,
                             sink=False, rot=rot, **kw)
        if spec.heads % spec.kv_heads:
            raise ValueError(f"layer {i}: heads {spec.heads} not a multiple of kv_heads {spec.kv_heads}")
        return spec

    for i, e in enumerate(raw):
        mx, kind = e["mixer"], e["type"]
        if kind == "attention":
            src = mx.get("kv_from")
            spec = attention(i, mx, "half", gate=True, gate_per_head=True, kv_from=None if src is None else int(src))
            if src is not None:
                o = raw[int(src)] if 0 <= int(src) < i else None
                if o is None or o["type"] != "attention" or o["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with its own cache")
                om = o["mixer"]
                if (int(om["heads"]), int(om.get("kv_heads", om["heads"])), int(om["dim"]), int(om.get("vdim", om["dim"]))) \
                        != (spec.heads, spec.kv_heads, spec.dim, spec.vdim):
                    raise ValueError(f"layer {i}: head shapes differ from layer {src}, whose keys and values it reads")
        elif kind == "parallel":
            L, R = mx["left"], mx["right"]
            left = attention(i, L, "interleaved", gate=False, qk_unit_norm=True, head_temp=True,
                             window=int(L["mask"]["size"]), pool=int(L["mask"]["pool"]))
            if left.window < 1 or left.pool < 1:
                raise ValueError(f"layer {i}: mask.size {left.window} and mask.pool {left.pool} must be at least 1")
            right = GatedRecurrenceSpec(width=int(R["width"]), blocks=int(R["blocks"]), conv=int(R["conv"]))
            if right.width % right.blocks or right.conv < 1:
                raise ValueError(f"layer {i}: width {right.width} in {right.blocks} blocks, {right.conv} taps")
            spec = SideBySideSpec(left=left, right=right, left_scale=float(mx["left_scale"]),
                                  right_scale=float(mx["right_scale"]))
        elif kind == "gla":
            spec = GatedLinearAttentionSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                                            tau=float(mx["tau"]), decay_rank=int(mx.get("decay_rank", 16)))
            if spec.tau <= 0:
                raise ValueError(f"layer {i}: tau {spec.tau} must be positive")
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = e.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            mlp = MLPSpec(kind="dense", ff=int(mlp["ff"]), act="clamped_swish", limit=float(mlp["limit"]))
        layers.append(LayerSpec(mixer=spec, mlp=mlp))
    taps = int((d.get("canon") or {}).get("taps", 0))
    if taps < 0:
        raise ValueError(f"canon.taps {taps}")
    eos_all = _eos_of(d)
    return LayerListConfig(architecture="Dotorax", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                           norm_eps=float(d["norm"]["eps"]), residual="sandwich", norm="rms_zero_centred",
                           residual_mult=float(d.get("residual_mult", 1.0)), canon_taps=taps, learned_positions=True,
                           max_position_embeddings=int(d["max_positions"]), eos_token_ids=eos_all,
                           eos_token_id=eos_all[0] if eos_all else None, bos_token_id=d.get("bos_token_id"))


def _dotorax_to_dict(c: "LayerListConfig") -> dict:
    def attention(m):
        mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
              "rot": m.rot.to_dict()}
        if m.kv_from is not None:
            mx["kv_from"] = m.kv_from
        if m.window:
            mx["mask"] = {"size": m.window, "pool": m.pool}
        return mx

    out = []
    for l in c.layers:
        m = l.mixer
        if m.kind == "attention":
            kind, mx = "attention", attention(m)
        elif m.kind == "side_by_side":
            kind = "parallel"
            mx = {"left": attention(m.left), "left_scale": m.left_scale, "right_scale": m.right_scale,
                  "right": {"width": m.right.width, "blocks": m.right.blocks, "conv": m.right.conv}}
        else:
            kind, mx = "gla", {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau, "decay_rank": m.decay_rank}
        mlp = None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff, "limit": l.mlp.limit}
        out.append({"type": kind, "mixer": mx, "mlp": mlp})
    return {"architecture": "Dotorax", "vocab": c.vocab_size, "width": c.hidden_size, "layers": out,
            "norm": {"eps": c.norm_eps}, "residual_mult": c.residual_mult, "canon": {"taps": c.canon_taps},
            "max_positions": c.max_position_embeddings}


# Named shapes used by tests and bench (random-init; there are no checkpoints offline).
def llama3_8b() -> ModelConfig:
    return ModelConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                       rope_theta=500000.0, max_position_embeddings=8192, eos_token_id=128001,
                       bos_token_id=128000)


def qwen2_05b() -> ModelConfig:
    """BASELINE.json configs[0] model shape (Qwen2-0.5B: q/k/v bias, tied embeddings, GQA group of 7)."""
    return ModelConfig(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                       num_attention_heads=14, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                       rope_theta=1e6, max_position_embeddings=32768, tie_word_embeddings=True,
                       attention_bias=True, architecture="Qwen2ForCausalLM", eos_token_id=151643,
                       bos_token_id=151643)


def llama3_70b() -> ModelConfig:
    return ModelConfig(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                       num_attention_heads=64, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                       rope_theta=500000.0, max_position_embeddings=8192, eos_token_id=128001,
                       bos_token_id=128000)


def tiny_mixtral() -> ModelConfig:
    return ModelConfig(vocab_size=512, hidden_size=512, intermediate_size=256, num_hidden_layers=2,
                       num_attention_heads=8, num_key_value_heads=2, head_dim=64, rope_theta=1e6,
                       max_position_embeddings=512, eos_token_id=2, bos_token_id=1,
                       architecture="MixtralForCausalLM", num_local_experts=8, num_experts_per_tok=2)


def mixtral_8x7b() -> ModelConfig:
    return ModelConfig(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                       rope_theta=1e6, max_position_embeddings=32768, eos_token_id=2, bos_token_id=1,
                       architecture="MixtralForCausalLM", num_local_experts=8, num_experts_per_tok=2)


def tiny_llama(head_dim: int = 64) -> ModelConfig:
    if head_dim == 128:
        return ModelConfig(vocab_size=640, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=1, head_dim=128,
                           max_position_embeddings=1024, eos_token_id=2, bos_token_id=1)
    return ModelConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                       num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                       max_position_embeddings=512, eos_token_id=2, bos_token_id=1)


@dataclass
class EngineConfig:
    model: str = ""
    served_model_name: Optional[str] = None
    max_model_len: Optional[int] = None
    tensor_parallel_size: int = 1
    gpu_memory_utilization: float = 0.90
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    num_gpu_blocks: Optional[int] = None      # override the memory-derived KV block count
    enforce_eager: bool = False               # skip CUDA-graph capture of decode steps
    enable_prefix_caching: bool = True        # reuse full KV blocks across requests (reference engine default)
    quantization: Optional[str] = None        # None | "fp8" (W8A8: online per-tensor weights, per-token activations)
    mixed_steps: bool = True                  # prefill steps also carry the running sequences' decode tokens
    kv_host_cache_gib: float = 0.0            # extended KV cache: pinned host memory for evicted prefix blocks (0 = off)
    # --speculative-config as a dict ({"method": "ngram", "num_speculative_tokens": k, ...}), None = off
    speculative_config: Optional[dict] = None
    seed: int = 0
    dtype: str = "bfloat16"                   # "float32": activations, caches and every product in true 32-bit
    #                                           (model families that have such a path; the others refuse it)
    max_logit_rows: Optional[int] = None      # rows of one step whose logits can be kept (default: one per sequence)
    block_size: int = 16
    cuda_graph_sizes: list = field(default_factory=list)

    def speculative(self):
        """Parsed speculative config, None when speculation is off or the method needs a draft model."""
        from .spec_decode import SpeculativeConfig

        c = SpeculativeConfig.parse(self.speculative_config)
        return c if (c is not None and c.supported) else None

    @property
    def num_speculative_tokens(self) -> int:
        c = self.speculative()
        return c.num_speculative_tokens if c is not None else 0

    def graph_buckets(self) -> list:
        if self.cuda_graph_sizes:
            return sorted(set(min(b, self.max_num_seqs) for b in self.cuda_graph_sizes))
        b = [1, 2, 4, 8]
        b += list(range(16, 129, 8))
        b += list(range(144, 513, 16))
        b += list(range(544, 1025, 32))
        b = [x for x in b if x <= self.max_num_seqs]
        if self.max_num_seqs not in b:
            b.append(self.max_num_seqs)
        return sorted(set(b))
