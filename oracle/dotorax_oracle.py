"""Plain, slow restatement of the Dotorax decoder -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

One function per mechanism, written from the design's equations in torch on the CPU, in one
floating-point type (float64 by default).  It shares nothing with gpustack_b200/: no kernels, no
cache, no scheduler; a sequence is processed whole, token by token where the design is a recurrence.

The design: x_0 = embed[token] + pos[p]; layers with a norm before AND after every sublayer,
x <- x + m * N_b(f(c(N_a(x)))), where N is an RMS norm whose weight is stored around zero (1 + w), c adds a
short causal per-channel convolution of the sublayer's input to that input, and f is the mixer or the
feed-forward.  Mixers: "attention" (grouped softmax attention, half-split rotation of the leading entries, a
sigmoid gate with ONE number per head, optionally on another layer's keys and values), "parallel" (a
sliding-window attention that also sees the mean key / value of every block of tokens that has wholly
left the window, beside a gated diagonal linear recurrence with a short convolution; the two outputs are
mixed with fixed factors) and "gla" (linear attention whose state rows decay with a data-dependent rate per
key channel).  The feed-forward is a clamped gated unit g sigmoid(1.702 g) (u + 1).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------ norms, activations
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------ short causal convolution
def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C] from a sequence's first token, w [C, taps] whose LAST column multiplies the current token:
    out_t = bias + sum_j w[:, j] x_(t - taps + 1 + j), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * x[s]
    return out if bias is None else out + bias


def input_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: its input plus the convolution of its input."""
    return h + causal_conv(h, w)


# ------------------------------------------------------------------------------ rotation
def rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int, layout: str) -> torch.Tensor:
    """x [T, heads, w]: the first `dims` entries of each head turn by position * base^(-2i/dims) in pair i;
    "half" pairs entry i with i + dims/2, "interleaved" pairs 2i with 2i+1."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    a = positions.to(x.dtype).reshape(-1, 1, 1) * f
    c, s = torch.cos(a), torch.sin(a)
    out = x.clone()
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half], out[..., half:dims] = u * c - v * s, v * c + u * s
    elif layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    else:
        raise ValueError(layout)
    return out


# ------------------------------------------------------------------------------ softmax attention
def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; head h reads key head h // (H / G); position i sees j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            p = torch.softmax((k[:i + 1, g] @ q[i, h]) * scale, dim=0)
            out[i, h] = p @ v[:i + 1, g]
    return out


def pooled_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: torch.Tensor, window: int,
                            pool: int) -> torch.Tensor:
    """Position i sees the tokens j with 0 <= i - j < window and, in the same softmax, one (mean key, mean value)
    for every block [b pool, (b + 1) pool) that ends at or before i - window.  scale [H]: a factor per head."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    nb_all = T // pool
    kb = k[:nb_all * pool].reshape(nb_all, pool, G, k.shape[2]).mean(dim=1)
    vb = v[:nb_all * pool].reshape(nb_all, pool, G, v.shape[2]).mean(dim=1)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            nb = max(0, (i - window + 1) // pool)          # blocks b with (b + 1) pool - 1 <= i - window
            keys = torch.cat([kb[:nb, g], k[lo:i + 1, g]], dim=0)
            vals = torch.cat([vb[:nb, g], v[lo:i + 1, g]], dim=0)
            p = torch.softmax((keys @ q[i, h]) * scale[h], dim=0)
            out[i, h] = p @ vals
    return out


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict,
                    kv: Optional[tuple] = None):
    """-> (output [T, D], (keys after rotation, values)).  kv: another layer's (keys, values) to read instead."""
    H, G, dk, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    rot = mx["rot"]
    q = rotate((h @ w["q"].T).reshape(T, H, dk), positions, float(rot["base"]), int(rot["dims"]), "half")
    if kv is None:
        k = rotate((h @ w["k"].T).reshape(T, G, dk), positions, float(rot["base"]), int(rot["dims"]), "half")
        v = (h @ w["v"].T).reshape(T, G, dv)
    else:
        k, v = kv
    o = causal_attention(q, k, v, float(mx["scale"]))
    gate = torch.sigmoid(h @ w["g"].T)                     # [T, H]
    o = o * gate.unsqueeze(-1)
    return o.reshape(T, H * dv) @ w["o"].T, (k, v)


# ------------------------------------------------------------------------------ gated diagonal recurrence
def gated_diagonal_recurrence(u: torch.Tensor, w: Dict[str, torch.Tensor], blocks: int) -> torch.Tensor:
    """u [T, C].  Per block of C / blocks channels: r = sigmoid(A_b u_b + a_b), i = sigmoid(B_b u_b + b_b);
    log a = -8 r softplus(lam); S_t = a S_(t-1) + sqrt(1 - a^2) i u, S before the first token = 0."""
    T, C = u.shape
    n = C // blocks
    ub = u.reshape(T, blocks, n)
    r = torch.sigmoid(torch.einsum("bon,tbn->tbo", w["ra"], ub) + w["ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("bon,tbn->tbo", w["ri"], ub) + w["ri.b"]).reshape(T, C)
    a = torch.exp(-8.0 * r * F.softplus(w["lam"]))
    x = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=u.dtype)
    out = torch.zeros_like(u)
    for t in range(T):
        S = a[t] * S + x[t]
        out[t] = S
    return out


def recurrent_branch(h: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict) -> torch.Tensor:
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    S = gated_diagonal_recurrence(u, w, int(mx["blocks"]))
    return (S * y) @ w["o"].T


def parallel_mixer(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict, eps: float) -> torch.Tensor:
    """w: names relative to the mixer ("left.q", "right.x", ...)."""
    L, R = mx["left"], mx["right"]
    H, G, dk, dv = int(L["heads"]), int(L["kv_heads"]), int(L["dim"]), int(L["vdim"])
    T = h.shape[0]
    rot = L["rot"]
    q = rotate((h @ w["left.q"].T).reshape(T, H, dk), positions, float(rot["base"]), int(rot["dims"]), "interleaved")
    k = rotate((h @ w["left.k"].T).reshape(T, G, dk), positions, float(rot["base"]), int(rot["dims"]), "interleaved")
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    v = (h @ w["left.v"].T).reshape(T, G, dv)
    o = pooled_window_attention(q, k, v, float(L["scale"]) * w["left.temp"], int(L["mask"]["size"]), int(L["mask"]["pool"]))
    left = o.reshape(T, H * dv) @ w["left.o"].T
    right = recurrent_branch(h, {n[6:]: t for n, t in w.items() if n.startswith("right.")}, R)
    return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right


# ------------------------------------------------------------------------------ gated linear attention
def gla_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict, eps: float) -> torch.Tensor:
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T (S: dk x dv, zero before the first token), o_t = S_t^T q_t,
    alpha = sigmoid(z)^(1/tau), z = A2 (A1 h) + b; o is normed per head (weight shared by the heads), gated by
    silu(G h) and projected."""
    H, dk, dv, tau = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"]), float(mx["tau"])
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.exp(F.logsigmoid(z) / tau).reshape(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_unit(o, eps) * w["norm"]
    return (o.reshape(T, H * dv) * silu(h @ w["g"].T)) @ w["o"].T


# ------------------------------------------------------------------------------ feed-forward
def clamped_gated_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


# ------------------------------------------------------------------------------ the model
def _sub(state: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t for n, t in state.items() if n.startswith(prefix)}


def forward(cfg: dict, state: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, trace: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; `trace` receives the residual after every layer."""
    w = {n: t.to(dtype) for n, t in state.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    kept: Dict[int, tuple] = {}
    for l, layer in enumerate(cfg["layers"]):
        p = f"l{l}."
        mx, kind = layer["mixer"], layer["type"]
        h = input_conv(zero_centred_rms_norm(x, w[p + "norm1"], eps), w[p + "canon1"])
        mw = _sub(w, p + "mix.")
        if kind == "attention":
            src = mx.get("kv_from")
            y, kv = attention_mixer(h, pos, mw, mx, None if src is None else kept[int(src)])
            if src is None:
                kept[l] = kv
        elif kind == "parallel":
            y = parallel_mixer(h, pos, mw, mx, eps)
        elif kind == "gla":
            y = gla_mixer(h, mw, mx, eps)
        else:
            raise ValueError(kind)
        x = x + m * zero_centred_rms_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = input_conv(zero_centred_rms_norm(x, w[p + "norm2"], eps), w[p + "canon2"])
            y = clamped_gated_ff(h, _sub(w, p + "mlp."), float(layer["mlp"]["limit"]))
            x = x + m * zero_centred_rms_norm(y, w[p + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return zero_centred_rms_norm(x, w["final.norm"], eps) @ w["head"].T


# ------------------------------------------------------------------------------ random models (tests)
def tensor_shapes(cfg: dict, decay_rank: int = 6) -> Dict[str, tuple]:
    """Tensor names and shapes of a checkpoint of this design; decay_rank: the rank of a gla mixer's decay projection
    (a checkpoint property: the configuration does not give it)."""
    D = int(cfg["width"])
    taps = int(cfg["canon"]["taps"])
    out: Dict[str, tuple] = {"embed": (int(cfg["vocab"]), D), "pos": (int(cfg["max_positions"]), D), "final.norm": (D,),
                             "head": (int(cfg["vocab"]), D)}

    def attention(p, mx, gate):
        H, G, dk, dv = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
        out[p + "q"] = (H * dk, D)
        if mx.get("kv_from") is None:
            out[p + "k"], out[p + "v"] = (G * dk, D), (G * dv, D)
        if gate:
            out[p + "g"] = (H, D)
        else:
            out[p + "temp"] = (H,)
        out[p + "o"] = (D, H * dv)

    for l, layer in enumerate(cfg["layers"]):
        p, mx = f"l{l}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (D,)
        out[p + "canon1"] = (D, taps)
        if layer["type"] == "attention":
            attention(p + "mix.", mx, True)
        elif layer["type"] == "parallel":
            attention(p + "mix.left.", mx["left"], False)
            R = mx["right"]
            W, B = int(R["width"]), int(R["blocks"])
            q = p + "mix.right."
            out[q + "y"] = out[q + "x"] = (W, D)
            out[q + "y.b"] = out[q + "x.b"] = out[q + "conv.b"] = out[q + "lam"] = (W,)
            out[q + "conv"] = (W, int(R["conv"]))
            out[q + "ra"] = out[q + "ri"] = (B, W // B, W // B)
            out[q + "ra.b"] = out[q + "ri.b"] = (B, W // B)
            out[q + "o"] = (D, W)
        else:
            H, dk, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
            q = p + "mix."
            out[q + "q"] = out[q + "k"] = (H * dk, D)
            out[q + "v"] = out[q + "g"] = (H * dv, D)
            out[q + "o"], out[q + "norm"] = (D, H * dv), (dv,)
            out[q + "a1"], out[q + "a2"], out[q + "a2.b"] = (decay_rank, D), (H * dk, decay_rank), (H * dk,)
        if layer.get("mlp") is not None:
            ff = int(layer["mlp"]["ff"])
            out[p + "norm2"] = out[p + "norm2b"] = (D,)
            out[p + "canon2"] = (D, taps)
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (ff, D)
            out[p + "mlp.down"] = (D, ff)
    return out


def random_weights(cfg: dict, seed: int = 0, decay_rank: int = 6) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights: linear weights N(0, 1 / in); norm weights around zero (the design stores them so) except the
    gla output norm around one; decays spread from fast to slow."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        x = torch.randn(tuple(shape), generator=g)
        leaf = name.split(".")[-1]
        if name.endswith("mix.norm"):
            x = 1.0 + 0.2 * x
        elif leaf.startswith("norm"):
            x = 0.25 * x
        elif leaf == "pos":
            x = 0.5 * x
        elif leaf in ("canon1", "canon2", "conv"):
            x = 0.5 * x
        elif leaf == "temp":
            x = 1.0 + 0.3 * x
        elif leaf == "lam":
            x = 1.5 * x - 1.0
        elif name.endswith("a2.b"):
            x = 2.0 + 1.5 * x
        elif name.endswith("a2"):
            x = 2.0 * x / math.sqrt(shape[-1])
        elif leaf == "b":
            x = 0.3 * x
        elif name != "embed":
            x = x / math.sqrt(shape[-1])
        out[name] = x.to(torch.bfloat16)
    return out
