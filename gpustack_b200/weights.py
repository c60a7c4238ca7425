"""Weight loading: HF-format safetensors directory -> fused, tensor-parallel-sharded bf16 (or
fp8 W8A8) tensors.

Sharding follows the reference engine's Megatron layout (SURVEY.md section 8e;
$VLLM/model_executor/models/llama.py:81-347): QKV and gate_up are column-parallel (each rank owns
Hq/t query heads, Hkv/t kv heads and I/t MLP columns), O and down are row-parallel (in-dim / t),
lm_head and the embedding table are vocab-parallel (rows [rank*ceil(V/t), ...)), the norms are replicated.

fp8 (`--quantization fp8`, or a checkpoint whose config.json carries quantization_config
{quant_method: fp8, activation_scheme: dynamic}): the four decoder linears of every layer are held
as e4m3 with ONE fp32 scale per fused weight, exactly as the reference engine prepares them --
bf16 checkpoints are quantised per tensor after fusing and sharding
($VLLM/model_executor/layers/quantization/fp8.py:537-549), per-tensor fp8 checkpoints are
re-quantised to the largest shard scale of a fused weight (fp8.py:406-428,
requantize_with_max_scale).  Embedding, norms and lm_head stay bf16.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

from .config import ModelConfig

BF16 = torch.bfloat16
FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
FP8_MIN_SCALE = 1.0 / (448.0 * 512.0)


@dataclass
class LayerWeights:
    input_norm: torch.Tensor      # [H]
    qkv: torch.Tensor             # [(Hq+2Hkv)/t * D, H]
    qkv_bias: Optional[torch.Tensor]
    o: torch.Tensor               # [H, Hq/t * D]
    post_norm: torch.Tensor       # [H]
    gate_up: Optional[torch.Tensor]   # [2I/t, H]  rows interleaved: 2i = gate_i, 2i+1 = up_i (fused SiLU*mul epilogue)
    down: Optional[torch.Tensor]      # [H, I/t]
    # fp8 mode: the four matrices above are float8_e4m3fn and these hold their fp32 scales ([1])
    qkv_scale: Optional[torch.Tensor] = None
    o_scale: Optional[torch.Tensor] = None
    gate_up_scale: Optional[torch.Tensor] = None
    down_scale: Optional[torch.Tensor] = None
    # Mixtral (gate_up / down are None): router replicated, experts stacked along the rows and
    # tensor-parallel over I exactly like the dense MLP
    router: Optional[torch.Tensor] = None      # [128, H]: E router rows, zero-padded to a GEMM tile
    w13: Optional[torch.Tensor] = None         # [E * 2I/t, H]  per expert: interleaved gate (w1) / up (w3) rows
    w2: Optional[torch.Tensor] = None          # [E * H, I/t]


@dataclass
class ModelWeights:
    embed: torch.Tensor           # [V/t, H]: this rank's vocabulary rows (the whole table when t == 1)
    layers: List[LayerWeights]
    final_norm: torch.Tensor      # [H]
    lm_head: torch.Tensor         # [V/t (padded to a multiple of 8), H]
    vocab_start: int
    vocab_end: int


def check_tp(cfg: ModelConfig, tp: int) -> None:
    # same divisibility rule the reference scheduler enforces
    # (gpustack/policies/candidate_selectors/base_candidate_selector.py:1007-1082)
    if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
        raise ValueError(f"tensor_parallel_size={tp} must divide attention heads "
                         f"({cfg.num_attention_heads}) and kv heads ({cfg.num_key_value_heads})")
    if cfg.intermediate_size % (tp * 64):
        raise ValueError(f"intermediate_size {cfg.intermediate_size} not divisible by 64*tp")


def quantize_fp8_per_tensor(w: torch.Tensor, scale: Optional[torch.Tensor] = None):
    """(e4m3 weight, fp32 scale[1]); scale = max(absmax/448, 1/(448*512)) unless given.  Load-time
    torch ops on the weight's device (same arithmetic as ops.scaled_fp8_quant(w, scale=None))."""
    wf = w.to(torch.float32)
    if scale is None:
        scale = (wf.abs().max() / FP8_MAX).clamp(min=FP8_MIN_SCALE)
    scale = scale.to(torch.float32).reshape(1)
    q = (wf * scale.reciprocal()).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.contiguous(), scale


def shard_state_dict(cfg: ModelConfig, get: Callable[[str], torch.Tensor], rank: int, tp: int,
                     device: str, quantization: Optional[str] = None,
                     has: Optional[Callable[[str], bool]] = None) -> ModelWeights:
    """`get(name)` returns the full HF tensor (any device); the result lives on `device`.
    quantization: None (bf16) or "fp8"; `has(name)` tells whether the checkpoint holds a tensor
    (needed to find `<proj>.weight_scale` / `.input_scale` of fp8 checkpoints)."""
    check_tp(cfg, tp)
    if quantization not in (None, "fp8"):
        raise ValueError(f"unsupported quantization {quantization!r} (supported: fp8)")
    D = cfg.head_dim
    hq, hkv, I = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp, cfg.intermediate_size // tp
    fp8 = quantization == "fp8"

    def dev(t):
        return t.to(device=device, dtype=BF16).contiguous()

    def shard_scale(name: str) -> Optional[torch.Tensor]:
        """per-tensor weight_scale of an fp8 checkpoint tensor, None for a bf16 one."""
        sname = name[: -len("weight")] + "weight_scale"
        if has is None or not has(sname):
            return None
        if has(name[: -len("weight")] + "input_scale"):
            raise ValueError("fp8 checkpoints with static activation scales are not supported "
                             "(activation_scheme must be dynamic)")
        sc = get(sname).to(torch.float32)
        if sc.numel() != 1:
            raise ValueError(f"{sname}: only per-tensor fp8 weight scales are supported")
        return sc.reshape(1).to(device)

    def fuse(names, slicers, interleave: bool = False):
        """Fused weight of this rank from the checkpoint tensors `names`, each cut by its slicer.
        bf16 mode -> (bf16 tensor, None); fp8 mode -> (e4m3 tensor, fp32 scale[1])."""
        parts = [sl(get(n)).to(device) for n, sl in zip(names, slicers)]
        scales = [shard_scale(n) for n in names] if fp8 else [None] * len(names)

        def merge(ts):
            if interleave:
                return torch.stack(ts, dim=1).reshape(2 * ts[0].shape[0], -1)
            return torch.cat(ts, dim=0) if len(ts) > 1 else ts[0]

        if not fp8:
            return dev(merge(parts)), None
        if all(sc is None for sc in scales):                      # online quantisation of a bf16 checkpoint
            return quantize_fp8_per_tensor(merge([p.to(BF16) for p in parts]))
        if any(sc is None for sc in scales) or any(p.dtype != FP8 for p in parts):
            raise ValueError(f"{names}: mixed fp8 / bf16 shards in one fused weight")
        if len(parts) == 1:
            return parts[0].contiguous(), scales[0]
        smax = torch.stack(scales).max().reshape(1)                # requantize_with_max_scale
        return quantize_fp8_per_tensor(merge([p.to(torch.float32) * sc for p, sc in zip(parts, scales)]), smax)

    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        qsl = lambda t: t[rank * hq * D:(rank + 1) * hq * D]          # noqa: E731
        ksl = lambda t: t[rank * hkv * D:(rank + 1) * hkv * D]        # noqa: E731
        isl = lambda t: t[rank * I:(rank + 1) * I]                    # noqa: E731
        bias = None
        if cfg.attention_bias:
            bias = dev(torch.cat([qsl(get(p + "self_attn.q_proj.bias")), ksl(get(p + "self_attn.k_proj.bias")),
                                  ksl(get(p + "self_attn.v_proj.bias"))]))
        qkv_w, qkv_s = fuse([p + f"self_attn.{n}_proj.weight" for n in "qkv"], [qsl, ksl, ksl])
        o_w, o_s = fuse([p + "self_attn.o_proj.weight"], [lambda t: t[:, rank * hq * D:(rank + 1) * hq * D]])
        moe = {}
        gu_w = gu_s = down_w = down_s = None
        if cfg.num_local_experts:
            if fp8:
                raise ValueError("fp8 quantisation of mixture-of-experts models is not supported yet")
            E = cfg.num_local_experts
            m = p + "block_sparse_moe."
            if has is not None and not has(m + "gate.weight") and has(p + "mlp.experts.gate_up_proj"):
                # transformers >= 5 export: experts fused as [E, 2I, H] (gate rows, then up rows) / [E, H, I]
                gup, dn = get(p + "mlp.experts.gate_up_proj"), get(p + "mlp.experts.down_proj")
                Ifull = cfg.intermediate_size
                w1 = [gup[e, :Ifull] for e in range(E)]
                w3 = [gup[e, Ifull:] for e in range(E)]
                w2 = [dn[e] for e in range(E)]
                router = get(p + "mlp.gate.weight")
            else:
                w1 = [get(m + f"experts.{e}.w1.weight") for e in range(E)]
                w3 = [get(m + f"experts.{e}.w3.weight") for e in range(E)]
                w2 = [get(m + f"experts.{e}.w2.weight") for e in range(E)]
                router = get(m + "gate.weight")
            w13 = torch.cat([torch.stack([isl(w1[e]).to(device), isl(w3[e]).to(device)], dim=1).reshape(2 * I, -1)
                             for e in range(E)], dim=0)
            router_pad = torch.zeros(128, router.shape[1], dtype=BF16)     # one full GEMM weight tile
            router_pad[:E] = router.to(BF16)
            moe = dict(router=dev(router_pad), w13=dev(w13),
                       w2=dev(torch.cat([w2[e][:, rank * I:(rank + 1) * I].to(device) for e in range(E)], dim=0)))
        else:
            gu_w, gu_s = fuse([p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], [isl, isl], interleave=True)
            down_w, down_s = fuse([p + "mlp.down_proj.weight"], [lambda t: t[:, rank * I:(rank + 1) * I]])
        layers.append(LayerWeights(
            input_norm=dev(get(p + "input_layernorm.weight")),
            qkv=qkv_w, qkv_bias=bias, o=o_w,
            post_norm=dev(get(p + "post_attention_layernorm.weight")),
            gate_up=gu_w, down=down_w,
            qkv_scale=qkv_s, o_scale=o_s, gate_up_scale=gu_s, down_scale=down_s, **moe))
    V = cfg.vocab_size
    per = (V + tp - 1) // tp
    v0, v1 = rank * per, min(V, (rank + 1) * per)
    # vocab-parallel embedding (VocabParallelEmbedding of the reference engine): each rank looks up
    # only its own rows, the partial result is summed by the first fused all-reduce + norm of the step
    embed = dev(get("model.embed_tokens.weight")[v0:v1])
    # tied embeddings: the lm_head shard IS the embedding shard (no second copy)
    lm = embed if cfg.tie_word_embeddings else dev(get("lm_head.weight")[v0:v1])
    return ModelWeights(embed=embed, layers=layers, final_norm=dev(get("model.norm.weight")),
                        lm_head=lm, vocab_start=v0, vocab_end=v1)


def load_safetensors_dir(cfg: ModelConfig, model_path: str, rank: int, tp: int, device: str,
                         quantization: Optional[str] = None) -> ModelWeights:
    from safetensors import safe_open

    root = Path(model_path)
    index = root / "model.safetensors.index.json"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
    else:
        weight_map = {}
        for f in sorted(root.glob("*.safetensors")):
            with safe_open(str(f), framework="pt") as sf:
                for k in sf.keys():
                    weight_map[k] = f.name
    if not weight_map:
        raise FileNotFoundError(f"no *.safetensors files under {model_path}")
    handles: Dict[str, object] = {}

    def get(name: str) -> torch.Tensor:
        fname = weight_map[name]
        if fname not in handles:
            handles[fname] = safe_open(str(root / fname), framework="pt")
        return handles[fname].get_tensor(name)

    return shard_state_dict(cfg, get, rank, tp, device, quantization=quantization,
                            has=lambda name: name in weight_map)


def random_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device: str = "cuda") -> Dict[str, torch.Tensor]:
    """Seeded N(0, std) bf16 weights in HF naming (synthetic checkpoints for benchmarks: no real
    weights exist offline).  Norm weights are 1 + N(0, 0.1)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def rnd(*shape, s=std):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * s).to(BF16)

    H, I = cfg.hidden_size, cfg.intermediate_size
    w = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H)}
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = (1.0 + rnd(H, s=0.1).float()).to(BF16)
        w[p + "self_attn.q_proj.weight"] = rnd(cfg.q_size, H)
        w[p + "self_attn.k_proj.weight"] = rnd(cfg.kv_size, H)
        w[p + "self_attn.v_proj.weight"] = rnd(cfg.kv_size, H)
        if cfg.attention_bias:
            for n, sz in (("q", cfg.q_size), ("k", cfg.kv_size), ("v", cfg.kv_size)):
                w[p + f"self_attn.{n}_proj.bias"] = rnd(sz)
        w[p + "self_attn.o_proj.weight"] = rnd(H, cfg.q_size)
        w[p + "post_attention_layernorm.weight"] = (1.0 + rnd(H, s=0.1).float()).to(BF16)
        if cfg.num_local_experts:
            w[p + "block_sparse_moe.gate.weight"] = rnd(cfg.num_local_experts, H, s=0.2)
            for e in range(cfg.num_local_experts):
                w[p + f"block_sparse_moe.experts.{e}.w1.weight"] = rnd(I, H)
                w[p + f"block_sparse_moe.experts.{e}.w3.weight"] = rnd(I, H)
                w[p + f"block_sparse_moe.experts.{e}.w2.weight"] = rnd(H, I)
            continue
        w[p + "mlp.gate_proj.weight"] = rnd(I, H)
        w[p + "mlp.up_proj.weight"] = rnd(I, H)
        w[p + "mlp.down_proj.weight"] = rnd(H, I)
    w["model.norm.weight"] = (1.0 + rnd(H, s=0.1).float()).to(BF16)
    if not cfg.tie_word_embeddings:
        w["lm_head.weight"] = rnd(cfg.vocab_size, H)
    return w


def lazy_random_source(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device: str = "cuda"):
    """(get, has) for shard_state_dict that synthesise each checkpoint tensor on demand instead of
    materialising the whole state dict first -- a 47 B-parameter Mixtral would otherwise be resident
    twice while its shards are fused.  Every tensor is N(0, std) (router 10x wider, norms 1 + N(0, 0.1))
    from a generator seeded by a hash of (seed, name), so any rank / any call order sees the same values."""
    import zlib

    H, I = cfg.hidden_size, cfg.intermediate_size
    shapes: Dict[str, tuple] = {"model.embed_tokens.weight": (cfg.vocab_size, H), "model.norm.weight": (H,)}
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (cfg.vocab_size, H)
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        shapes[p + "input_layernorm.weight"] = (H,)
        shapes[p + "post_attention_layernorm.weight"] = (H,)
        for n, rows in (("q", cfg.q_size), ("k", cfg.kv_size), ("v", cfg.kv_size)):
            shapes[p + f"self_attn.{n}_proj.weight"] = (rows, H)
            if cfg.attention_bias:
                shapes[p + f"self_attn.{n}_proj.bias"] = (rows,)
        shapes[p + "self_attn.o_proj.weight"] = (H, cfg.q_size)
        if cfg.num_local_experts:
            shapes[p + "block_sparse_moe.gate.weight"] = (cfg.num_local_experts, H)
            for e in range(cfg.num_local_experts):
                shapes[p + f"block_sparse_moe.experts.{e}.w1.weight"] = (I, H)
                shapes[p + f"block_sparse_moe.experts.{e}.w3.weight"] = (I, H)
                shapes[p + f"block_sparse_moe.experts.{e}.w2.weight"] = (H, I)
        else:
            shapes[p + "mlp.gate_proj.weight"] = (I, H)
            shapes[p + "mlp.up_proj.weight"] = (I, H)
            shapes[p + "mlp.down_proj.weight"] = (H, I)

    def get(name: str) -> torch.Tensor:
        g = torch.Generator(device=device)
        g.manual_seed(zlib.crc32(f"{seed}/{name}".encode()) | (zlib.crc32(f"{name}#{seed}".encode()) << 32))
        shape = shapes[name]
        x = torch.randn(*shape, generator=g, device=device, dtype=torch.float32)
        if name.endswith("norm.weight"):
            return (1.0 + x * 0.1).to(BF16)
        return (x * (10 * std if name.endswith("block_sparse_moe.gate.weight") else std)).to(BF16)

    return get, (lambda name: name in shapes)


def save_checkpoint(cfg: ModelConfig, state: Dict[str, torch.Tensor], out_dir: str, shard_bytes: int = 4 << 30) -> None:
    """Write an HF-format directory (config.json + sharded safetensors + index) so that the same
    synthetic weights can be served by this engine and by the reference's vLLM backend."""
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg.to_hf_dict(), indent=1))
    shards, cur, cur_bytes = [], {}, 0
    for k, v in state.items():
        n = v.numel() * v.element_size()
        if cur and cur_bytes + n > shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v.detach().to("cpu").contiguous()
        cur_bytes += n
    if cur:
        shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, str(out / name), metadata={"format": "pt"})
        for k in sh:
            weight_map[k] = name
    (out / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {}, "weight_map": weight_map}, indent=1))


# ------------------------------------------------------------------------------ layer-list designs
@dataclass
class LayerListLayer:
    """One layer of a layer-list decoder.  Everything that reads the mixer's input is ONE fused projection:
    attention  rows = [q: H*dk | k: G*dk | v: G*dv | gate: H*dv]   (no k / v rows with kv_from),
    mlstm      rows = [q: H*dk | k: H*dk | v: H*dv | gate: H*dv];  its two per-head gate projections are a
    second, fp32-output projection `gates` = [input: H | forget: H],
    linear attention  rows = [q: H*dk | k: H*dk | v: H*dv | gate: H*dv]; an attention mixer whose values are its
    keys has no v rows."""
    norm1: torch.Tensor
    proj: torch.Tensor
    o: torch.Tensor
    proj_bias: Optional[torch.Tensor] = None     # attention: bias of the q (, k, v) rows
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    sink: Optional[torch.Tensor] = None          # [H] fp32
    gates: Optional[torch.Tensor] = None         # mlstm: [2H, D]
    gate_bias: Optional[torch.Tensor] = None     # mlstm: [2H]
    out_norm: Optional[torch.Tensor] = None      # mlstm: [H*dv]
    norm2: Optional[torch.Tensor] = None
    up: Optional[torch.Tensor] = None
    down: Optional[torch.Tensor] = None
    # tanh norm: bias vector and the scalar alpha (fp32 [1]) of norm1 / norm2
    norm1_b: Optional[torch.Tensor] = None
    norm1_alpha: Optional[torch.Tensor] = None
    norm2_b: Optional[torch.Tensor] = None
    norm2_alpha: Optional[torch.Tensor] = None
    # residual streams: per sublayer ONE fp32 vector [in: s | out: s | mix: s*s (from, to)]
    hc1: Optional[torch.Tensor] = None
    hc2: Optional[torch.Tensor] = None
    # latent attention: proj rows = [q: H*(dim+rot_dim)  or  query latent: q_rank | latent: kv_rank | key part: rot_dim]
    q_lat_norm: Optional[torch.Tensor] = None    # [q_rank]
    uq: Optional[torch.Tensor] = None            # [H*(dim+rot_dim), q_rank]
    kv_norm: Optional[torch.Tensor] = None       # [kv_rank]
    uk_t: Optional[torch.Tensor] = None          # [H, kv_rank, dim]: W_uk of each head transposed (query absorption)
    uv: Optional[torch.Tensor] = None            # [H*vdim, kv_rank]
    rot_freq: Optional[torch.Tensor] = None      # fp64 [dims/2]: angular frequency of every rotated pair
    rot_mag: float = 1.0                         # factor on cos and sin (frequency-scaled rotations)
    decay: Optional[torch.Tensor] = None         # linear attention: fp32 [H], the per-head decay
    # gated feed-forward: gate_up rows interleaved (2i = gate_i, 2i+1 = up_i), `up` above is unused
    gate_up: Optional[torch.Tensor] = None       # [2 ff, D]
    # routed feed-forward
    router: Optional[torch.Tensor] = None        # [experts + identity rounded up to 128, D], zero rows behind the outputs
    correction: Optional[torch.Tensor] = None    # fp32 [experts + identity]
    w13: Optional[torch.Tensor] = None           # [experts * 2 ff, D], per expert interleaved gate / up rows
    w2: Optional[torch.Tensor] = None            # [experts * D, ff]
    shared13: Optional[torch.Tensor] = None      # [2 shared_ff, D]
    shared2: Optional[torch.Tensor] = None       # [D, shared_ff]
    # sandwich residual: the norms after the mixer and after the feed-forward
    norm1b: Optional[torch.Tensor] = None
    norm2b: Optional[torch.Tensor] = None
    # input convolution of the mixer / the feed-forward: fp32 [D, taps]
    canon1: Optional[torch.Tensor] = None
    canon2: Optional[torch.Tensor] = None
    head_scale: Optional[torch.Tensor] = None    # attention: fp32 [H], a factor per head on the score
    # side-by-side mixer: proj rows = [q | k | v (left attention) | y | x (recurrent branch)], zero rows up to a multiple
    # of 8; `o` is the left output projection, `o2` the right one
    o2: Optional[torch.Tensor] = None
    rec_bias: Optional[torch.Tensor] = None      # fp32 [2 W]: biases of the y and x rows
    rec_conv: Optional[torch.Tensor] = None      # fp32 [W, taps]
    rec_conv_bias: Optional[torch.Tensor] = None  # fp32 [W]
    rec_gates: Optional[torch.Tensor] = None     # bf16 [2 * blocks, n, n]: the recurrence gate's blocks, then the input gate's
    rec_gate_bias: Optional[torch.Tensor] = None  # fp32 [2 W]
    rec_lam: Optional[torch.Tensor] = None       # fp32 [W]
    # gated linear attention: proj rows = [q | k | v | gate | decay latent]; the decay's second projection and bias
    decay_up: Optional[torch.Tensor] = None      # bf16 [H*dk, rank]
    decay_bias: Optional[torch.Tensor] = None    # bf16 [H*dk]


@dataclass
class LayerListWeights:
    embed: torch.Tensor
    layers: List[LayerListLayer]
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    vocab_start: int = 0
    vocab_end: int = 0
    final_norm_b: Optional[torch.Tensor] = None
    final_norm_alpha: Optional[torch.Tensor] = None
    pos: Optional[torch.Tensor] = None           # learned positions [max_position_embeddings, D]


def layer_list_tensor_shapes(cfg) -> Dict[str, tuple]:
    """Checkpoint tensor names and shapes of a layer-list model (linear weights are [out, in])."""
    D = cfg.hidden_size
    shapes: Dict[str, tuple] = {"embed": (cfg.vocab_size, D), "final.norm": (D,), "head": (cfg.vocab_size, D)}
    tanh = getattr(cfg, "norm", "layernorm") == "tanh"
    S = getattr(cfg, "streams", 0)
    parallel = getattr(cfg, "residual", "post_ln") == "parallel"     # one norm per layer feeds both sublayers

    def norm_shapes(name):
        shapes[name] = (D,)
        if tanh:
            shapes[name + ".b"] = (D,)
            shapes[name + ".alpha"] = ()

    if tanh:
        norm_shapes("final.norm")
    sandwich = getattr(cfg, "residual", "post_ln") == "sandwich"
    taps = getattr(cfg, "canon_taps", 0)
    if getattr(cfg, "learned_positions", False):
        shapes["pos"] = (cfg.max_position_embeddings, D)

    def attention_shapes(q, m):
        shapes[q + "q"] = (m.q_width, D)
        if m.kv_from is None:
            shapes[q + "k"], shapes[q + "v"] = (m.kv_heads * m.dim, D), (m.kv_heads * m.vdim, D)
        if m.gate:
            shapes[q + "g"] = (m.gate_width, D)
        if m.head_temp:
            shapes[q + "temp"] = (m.heads,)
        shapes[q + "o"] = (D, m.out_width)

    for l, layer in enumerate(cfg.layers):
        p, m = f"l{l}.", layer.mixer
        norm_shapes(p + "norm1")
        if sandwich:
            shapes[p + "norm1b"] = (D,)
            if taps:
                shapes[p + "canon1"] = (D, taps)
            if m.kind == "attention":
                attention_shapes(p + "mix.", m)
            elif m.kind == "side_by_side":
                attention_shapes(p + "mix.left.", m.left)
                r, q = m.right, p + "mix.right."
                n = r.width // r.blocks
                for b_ in ("y", "x"):
                    shapes[q + b_], shapes[q + b_ + ".b"] = (r.width, D), (r.width,)
                shapes[q + "conv"], shapes[q + "conv.b"] = (r.width, r.conv), (r.width,)
                for g_ in ("ra", "ri"):
                    shapes[q + g_], shapes[q + g_ + ".b"] = (r.blocks, n, n), (r.blocks, n)
                shapes[q + "lam"], shapes[q + "o"] = (r.width,), (D, r.width)
            else:
                q = p + "mix."
                shapes[q + "q"] = shapes[q + "k"] = (m.heads * m.dim, D)
                shapes[q + "v"] = shapes[q + "g"] = (m.out_width, D)
                shapes[q + "o"], shapes[q + "norm"] = (D, m.out_width), (m.vdim,)
                shapes[q + "a1"], shapes[q + "a2"], shapes[q + "a2.b"] = (m.decay_rank, D), (m.heads * m.dim, m.decay_rank), \
                    (m.heads * m.dim,)
            if layer.mlp is not None:
                shapes[p + "norm2"] = shapes[p + "norm2b"] = (D,)
                if taps:
                    shapes[p + "canon2"] = (D, taps)
                shapes[p + "mlp.gate"] = shapes[p + "mlp.up"] = (layer.mlp.ff, D)
                shapes[p + "mlp.down"] = (D, layer.mlp.ff)
            continue
        for q in ((1, 2) if layer.mlp is not None else (1,)) if S else ():
            shapes[p + f"hc{q}.in"], shapes[p + f"hc{q}.out"], shapes[p + f"hc{q}.mix"] = (S,), (S,), (S, S)
        if m.kind == "latent_attention":
            if m.q_rank:
                shapes[p + "mix.dq"], shapes[p + "mix.dq.norm"] = (m.q_rank, D), (m.q_rank,)
                shapes[p + "mix.uq"] = (m.q_width, m.q_rank)
            else:
                shapes[p + "mix.q"] = (m.q_width, D)
            shapes[p + "mix.dkv"], shapes[p + "mix.dkv.norm"] = (m.cache_width, D), (m.kv_rank,)
            shapes[p + "mix.uk"] = (m.heads * m.dim, m.kv_rank)
            shapes[p + "mix.uv"] = (m.out_width, m.kv_rank)
            if m.sink:
                shapes[p + "mix.sink"] = (m.heads,)
            shapes[p + "mix.o"] = (D, m.out_width)
        elif m.kind == "attention":
            shapes[p + "mix.q"] = (m.q_width, D)
            if m.qkv_bias:
                shapes[p + "mix.q.b"] = (m.q_width,)
            if m.qk_norm:
                shapes[p + "mix.q.norm"] = (m.dim,)
            if m.kv_from is None:
                shapes[p + "mix.k"] = (m.kv_heads * m.dim, D)
                if not m.values_are_keys:
                    shapes[p + "mix.v"] = (m.kv_heads * m.vdim, D)
                if m.qkv_bias:
                    shapes[p + "mix.k.b"] = (m.kv_heads * m.dim,)
                    shapes[p + "mix.v.b"] = (m.kv_heads * m.vdim,)
                if m.qk_norm:
                    shapes[p + "mix.k.norm"] = (m.dim,)
            if m.sink:
                shapes[p + "mix.sink"] = (m.heads,)
            if m.gate:
                shapes[p + "mix.g"] = (m.out_width, D)
            shapes[p + "mix.o"] = (D, m.out_width)
        elif m.kind == "linear_attention":
            for n, rows in (("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.out_width), ("g", m.out_width)):
                shapes[p + "mix." + n] = (rows, D)
            shapes[p + "mix.o"] = (D, m.out_width)
            if m.out_norm == "all_heads":
                shapes[p + "mix.norm"] = (m.out_width,)
        else:
            for n, rows in (("q", m.heads * m.dim), ("k", m.heads * m.dim), ("v", m.out_width), ("g", m.out_width)):
                shapes[p + "mix." + n] = (rows, D)
            shapes[p + "mix.o"] = (D, m.out_width)
            shapes[p + "mix.norm"] = (m.out_width,)
            for n in ("i", "f"):
                shapes[p + "mix." + n] = (m.heads, D)
                shapes[p + "mix." + n + ".b"] = (m.heads,)
        if layer.mlp is not None:
            if not parallel:
                norm_shapes(p + "norm2")
            if layer.mlp.kind == "moe":
                e = layer.mlp.moe
                for i in range(e.experts):
                    shapes[p + f"mlp.e{i}.gate"] = shapes[p + f"mlp.e{i}.up"] = (e.ff, D)
                    shapes[p + f"mlp.e{i}.down"] = (D, e.ff)
                shapes[p + "mlp.router"] = (e.experts + e.identity, D)
                if e.score == "softmax":
                    shapes[p + "mlp.correction"] = (e.experts + e.identity,)
                if e.shared_ff:
                    shapes[p + "mlp.shared.gate"] = shapes[p + "mlp.shared.up"] = (e.shared_ff, D)
                    shapes[p + "mlp.shared.down"] = (D, e.shared_ff)
                continue
            if layer.mlp.act != "relu2":
                shapes[p + "mlp.gate"] = (layer.mlp.ff, D)
            shapes[p + "mlp.up"] = (layer.mlp.ff, D)
            shapes[p + "mlp.down"] = (D, layer.mlp.ff)
    return shapes


def _interleave_rows(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[n, K] gate and up rows -> [2n, K] with row 2i = gate_i, row 2i+1 = up_i (the layout of the gated epilogues)."""
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()


def load_layer_list(cfg, get: Callable[[str], torch.Tensor], device: str) -> LayerListWeights:
    """Fuse the checkpoint tensors of a layer-list model (names as layer_list_tensor_shapes) on `device`.
    Weights stay bf16 whatever the serving precision: a 32-bit model converts them exactly on the fly."""
    shapes = layer_list_tensor_shapes(cfg)

    def g(name: str) -> torch.Tensor:
        t = get(name)
        if tuple(t.shape) != shapes[name]:
            raise ValueError(f"{name}: shape {tuple(t.shape)} does not match the config ({shapes[name]})")
        return t.to(device=device, dtype=BF16)

    def cat(names):
        return torch.cat([g(n) for n in names], dim=0).contiguous()

    def f32(name: str) -> torch.Tensor:
        return g(name).to(torch.float32).reshape(-1).contiguous()

    tanh = getattr(cfg, "norm", "layernorm") == "tanh"
    S = getattr(cfg, "streams", 0)
    parallel = getattr(cfg, "residual", "post_ln") == "parallel"

    def hyper(prefix: str) -> torch.Tensor:
        if not S:        # one plain residual stream: read it, keep it, add the branch
            return torch.ones(3, dtype=torch.float32, device=device)
        return torch.cat([f32(prefix + ".in"), f32(prefix + ".out"), f32(prefix + ".mix")]).contiguous()

    def cat8(names):
        """Fused projection rows, zero rows up to a multiple of 8 (16-byte output rows for the tensor-core GEMM)."""
        w = cat(names)
        pad = -w.shape[0] % 8
        return w if not pad else torch.cat([w, torch.zeros(pad, w.shape[1], dtype=BF16, device=device)]).contiguous()

    def freq_of(rot):
        return torch.tensor(list(rot.frequencies()[0]), dtype=torch.float64).to(device)

    layers = []
    for l, layer in enumerate(cfg.layers):
        p, m = f"l{l}.", layer.mixer
        if getattr(cfg, "residual", "post_ln") == "sandwich":
            q = p + "mix."
            if m.kind == "attention":
                own = m.kv_from is None
                lw = LayerListLayer(norm1=g(p + "norm1"), o=g(q + "o"),
                                    proj=cat8([q + n for n in ["q"] + (["k", "v"] if own else []) + (["g"] if m.gate else [])]))
                lw.rot_freq = freq_of(m.rot)
            elif m.kind == "side_by_side":
                a, r = m.left, m.right
                lw = LayerListLayer(norm1=g(p + "norm1"), o=g(q + "left.o"), o2=g(q + "right.o"),
                                    proj=cat8([q + "left.q", q + "left.k", q + "left.v", q + "right.y", q + "right.x"]))
                lw.rot_freq = freq_of(a.rot)
                lw.head_scale = f32(q + "left.temp") if a.head_temp else None
                lw.rec_bias = torch.cat([f32(q + "right.y.b"), f32(q + "right.x.b")]).contiguous()
                lw.rec_conv = g(q + "right.conv").to(torch.float32).contiguous()
                lw.rec_conv_bias = f32(q + "right.conv.b")
                lw.rec_gates = torch.cat([g(q + "right.ra"), g(q + "right.ri")], dim=0).contiguous()
                lw.rec_gate_bias = torch.cat([f32(q + "right.ra.b"), f32(q + "right.ri.b")]).contiguous()
                lw.rec_lam = f32(q + "right.lam")
            else:
                a1 = get(q + "a1")
                m.decay_rank = int(a1.shape[0])          # the checkpoint decides the rank of the decay's latent
                shapes.update(layer_list_tensor_shapes(cfg))
                lw = LayerListLayer(norm1=g(p + "norm1"), o=g(q + "o"), out_norm=g(q + "norm"),
                                    proj=cat8([q + n for n in ("q", "k", "v", "g", "a1")]))
                lw.decay_up, lw.decay_bias = g(q + "a2"), g(q + "a2.b")
            lw.norm1b = g(p + "norm1b")
            if getattr(cfg, "canon_taps", 0):
                lw.canon1 = g(p + "canon1").to(torch.float32).contiguous()
            if layer.mlp is not None:
                lw.norm2, lw.norm2b = g(p + "norm2"), g(p + "norm2b")
                if getattr(cfg, "canon_taps", 0):
                    lw.canon2 = g(p + "canon2").to(torch.float32).contiguous()
                lw.gate_up, lw.down = _interleave_rows(g(p + "mlp.gate"), g(p + "mlp.up")), g(p + "mlp.down")
            layers.append(lw)
            continue
        if m.kind == "latent_attention":
            first = g(p + "mix.dq") if m.q_rank else g(p + "mix.q")
            lw = LayerListLayer(norm1=g(p + "norm1"), proj=torch.cat([first, g(p + "mix.dkv")], dim=0).contiguous(),
                                o=g(p + "mix.o"))
            if m.q_rank:
                lw.q_lat_norm, lw.uq = g(p + "mix.dq.norm"), g(p + "mix.uq")
            lw.kv_norm = g(p + "mix.dkv.norm")
            lw.uk_t = g(p + "mix.uk").view(m.heads, m.dim, m.kv_rank).transpose(1, 2).contiguous()
            lw.uv = g(p + "mix.uv")
            if m.sink:
                lw.sink = f32(p + "mix.sink")
            freqs, mag = m.rot.frequencies()
            lw.rot_freq, lw.rot_mag = torch.tensor(list(freqs), dtype=torch.float64).to(device), float(mag)
        elif m.kind == "attention":
            own = m.kv_from is None
            names = ["q"] + ((["k"] if m.values_are_keys else ["k", "v"]) if own else []) + (["g"] if m.gate else [])
            lw = LayerListLayer(norm1=g(p + "norm1"), proj=cat([p + "mix." + n for n in names]), o=g(p + "mix.o"))
            if m.qkv_bias:
                lw.proj_bias = cat([p + f"mix.{n}.b" for n in (["q", "k", "v"] if own else ["q"])])
            if m.qk_norm:
                lw.q_norm = g(p + "mix.q.norm")
                lw.k_norm = g(p + "mix.k.norm") if own else None
            if m.sink:
                lw.sink = g(p + "mix.sink").to(torch.float32).contiguous()
            if m.rot is not None:
                lw.rot_freq = torch.tensor(list(m.rot.frequencies()[0]), dtype=torch.float64).to(device)
        elif m.kind == "linear_attention":
            lw = LayerListLayer(norm1=g(p + "norm1"), proj=cat([p + "mix." + n for n in "qkvg"]), o=g(p + "mix.o"))
            if m.out_norm == "all_heads":
                lw.out_norm = g(p + "mix.norm")
            lw.decay = torch.tensor(list(m.decay), dtype=torch.float32).to(device)
            if m.rot is not None:
                lw.rot_freq = torch.tensor(list(m.rot.frequencies()[0]), dtype=torch.float64).to(device)
        else:
            lw = LayerListLayer(norm1=g(p + "norm1"), proj=cat([p + "mix." + n for n in "qkvg"]), o=g(p + "mix.o"),
                                gates=cat([p + "mix.i", p + "mix.f"]), gate_bias=cat([p + "mix.i.b", p + "mix.f.b"]),
                                out_norm=g(p + "mix.norm"))
        if tanh:
            lw.norm1_b, lw.norm1_alpha = g(p + "norm1.b"), f32(p + "norm1.alpha")
        if getattr(cfg, "residual", "post_ln") == "streams":
            lw.hc1 = hyper(p + "hc1")
        if layer.mlp is not None:
            if not parallel:
                lw.norm2 = g(p + "norm2")
            if tanh:
                lw.norm2_b, lw.norm2_alpha = g(p + "norm2.b"), f32(p + "norm2.alpha")
            if getattr(cfg, "residual", "post_ln") == "streams":
                lw.hc2 = hyper(p + "hc2")
            if layer.mlp.kind == "moe":
                e = layer.mlp.moe
                # zero rows up to a whole GEMM weight tile: the router projection is an ordinary one-tile product
                router = g(p + "mlp.router")
                lw.router = torch.zeros(-(-router.shape[0] // 128) * 128, router.shape[1], dtype=BF16, device=device)
                lw.router[:router.shape[0]] = router
                lw.correction = f32(p + "mlp.correction") if e.score == "softmax" else None
                lw.w13 = torch.cat([_interleave_rows(g(p + f"mlp.e{i}.gate"), g(p + f"mlp.e{i}.up"))
                                    for i in range(e.experts)], dim=0).contiguous()
                lw.w2 = torch.cat([g(p + f"mlp.e{i}.down") for i in range(e.experts)], dim=0).contiguous()
                if e.shared_ff:
                    lw.shared13 = _interleave_rows(g(p + "mlp.shared.gate"), g(p + "mlp.shared.up"))
                    lw.shared2 = g(p + "mlp.shared.down")
            elif layer.mlp.act == "relu2":
                lw.up, lw.down = g(p + "mlp.up"), g(p + "mlp.down")
            else:
                lw.gate_up, lw.down = _interleave_rows(g(p + "mlp.gate"), g(p + "mlp.up")), g(p + "mlp.down")
        layers.append(lw)
    out = LayerListWeights(embed=g("embed"), layers=layers, final_norm=g("final.norm"), lm_head=g("head"),
                           vocab_start=0, vocab_end=cfg.vocab_size)
    if tanh:
        out.final_norm_b, out.final_norm_alpha = g("final.norm.b"), f32("final.norm.alpha")
    if getattr(cfg, "learned_positions", False):
        out.pos = g("pos")
    return out


def load_layer_list_dir(cfg, model_path: str, device: str) -> LayerListWeights:
    from safetensors import safe_open

    files = sorted(Path(model_path).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no *.safetensors files under {model_path}")
    where: Dict[str, object] = {}
    for f in files:
        h = safe_open(str(f), framework="pt")
        for k in h.keys():
            where[k] = h
    return load_layer_list(cfg, lambda name: where[name].get_tensor(name), device)


def random_layer_list_state(cfg, seed: int = 0, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Seeded bf16 checkpoint of a layer-list model (benchmarks and tests: no trained weights exist).
    Linear weights N(0, 1/in), biases and sinks of order 1, norm weights 1 + N(0, 0.2), forget-gate
    biases around +3 so that the recurrent state keeps a long memory."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in layer_list_tensor_shapes(cfg).items():
        x = torch.randn(tuple(shape), generator=gen, device=device, dtype=torch.float32)
        leaf = name.split(".", 1)[1] if name[0] == "l" and name[1].isdigit() else name
        if leaf.endswith(".alpha"):
            x = 0.5 + 0.1 * x
        elif leaf.endswith("norm.b") or leaf in ("norm1.b", "norm2.b"):
            x = 0.1 * x
        elif leaf.endswith(".mix") and leaf.startswith("hc"):
            x = torch.eye(shape[0], device=device) * 0.8 + 0.15 * x
        elif leaf.startswith("hc"):
            x = 0.7 + 0.2 * x
        elif leaf == "mlp.correction":
            x = 0.05 * x
        elif getattr(cfg, "norm", "") == "rms_zero_centred" and (leaf.endswith("norm") or leaf[:5] in ("norm1", "norm2")) \
                and leaf != "mix.norm":
            x = 0.2 * x                                   # stored around zero
        elif leaf == "pos":
            x = 0.5 * x
        elif leaf in ("canon1", "canon2"):
            x = 0.4 * x
        elif leaf.endswith(".temp"):
            x = 1.0 + 0.3 * x
        elif leaf.endswith(".lam"):
            x = -1.0 + x                                  # decays spread between fast and slow
        elif leaf.endswith(".conv"):
            x = 0.5 * x
        elif leaf.endswith(".ra") or leaf.endswith(".ri"):
            x = x / (shape[-1] ** 0.5)
        elif leaf == "mix.a2.b":
            x = 2.0 + x                                   # sigmoid(z) mostly near one: a long memory
        elif leaf.endswith("norm") or leaf in ("norm1", "norm2"):
            x = 1.0 + 0.2 * x
        elif leaf == "mix.f.b":
            x = 3.0 + x
        elif leaf == "mix.sink":
            x = 1.5 * x
        elif leaf.endswith(".b"):
            x = 0.3 * x if leaf != "mix.i.b" else x
        elif leaf == "embed":
            pass
        else:
            x = x / (shape[-1] ** 0.5) if len(shape) else x
        out[name] = x.to(BF16)
    return out


def save_layer_list_checkpoint(cfg, state: Dict[str, torch.Tensor], out_dir: str) -> None:
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    save_file({k: v.detach().to("cpu").contiguous() for k, v in state.items()}, str(out / "model.safetensors"))
