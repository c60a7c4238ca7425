"""Plain, slow restatement of the Resevik decoder -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

One function per mechanism, written from the design's equations in torch on the CPU, in one
floating-point type (float64 by default).  It shares nothing with gpustack_b200/: no kernels, no
cache, no scheduler; a sequence is processed whole, token by token where the design is a recurrence.

The design: pre-norm layers in which ONE RMS norm feeds the mixer and the feed-forward side by side
(x <- x + mixer(h) + ff(h), h = norm(x)); three mixers -- decayed linear attention with SiLU feature
maps and a sigmoid gate ("lightning"), decayed linear attention with half-split rotation and a SiLU
gate ("retention"), and sliding-window softmax attention whose values are the unrotated keys, with
interleaved rotation followed by a weightless RMS norm of q and k ("attention"); a routed
feed-forward with sigmoid scores that multiply the chosen experts' INPUT; a span of layers that is run
several times with the same weights (every pass with its own cache / state, the embedding added
again before each repeated pass).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------ norms, activations
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------ rotation
def rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int, layout: str) -> torch.Tensor:
    """x [T, heads, w]: the first `dims` entries of every head are rotated by the angle position * base^(-2i/dims)
    of pair i; 'interleaved' pairs (2i, 2i+1), 'half' pairs (i, i + dims/2).  The rest pass unchanged."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = base ** (-2.0 * i / dims)
    a = positions.to(x.dtype).reshape(-1, 1, 1) * f
    c, s = torch.cos(a), torch.sin(a)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    elif layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


# ------------------------------------------------------------------------------ softmax attention
def window_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence from position 0; query head h reads key head
    h // (H / G); position i sees j with 0 <= i - j < window.  -> [T, H, dv]"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict, eps: float) -> torch.Tensor:
    """Values are the keys as projected; q and k are rotated (interleaved pairs), then divided by their root mean
    square per head; sliding window; output projection."""
    H, G, dk = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"])
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dk)
    k = (h @ w["k"].T).reshape(T, G, dk)
    v = k.clone()
    rot = mx["rot"]
    q = rms_norm(rotate(q, positions, float(rot["base"]), int(rot["dims"]), "interleaved"), None, eps)
    k = rms_norm(rotate(k, positions, float(rot["base"]), int(rot["dims"]), "interleaved"), None, eps)
    o = window_softmax_attention(q, k, v, float(mx["scale"]), int(mx["mask"]["size"]))
    return o.reshape(T, -1) @ w["o"].T


# ------------------------------------------------------------------------------ decayed linear attention
def decayed_linear_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                             state: Optional[torch.Tensor] = None):
    """Per head  S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t.  q, k [T, H, dk], v [T, H, dv], decay [H];
    state [H, dk, dv] (None = zero).  -> (o [T, H, dv], the state after the last token)"""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = decay.reshape(H, 1, 1) * S + k[t].unsqueeze(2) * v[t].unsqueeze(1)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def lightning_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict, eps: float) -> torch.Tensor:
    """SiLU on q, k and v; all heads normed together (RMS, with a weight); sigmoid gate; output projection."""
    H, dk, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    q = silu(h @ w["q"].T).reshape(T, H, dk)
    k = silu(h @ w["k"].T).reshape(T, H, dk)
    v = silu(h @ w["v"].T).reshape(T, H, dv)
    o, _ = decayed_linear_attention(q, k, v, torch.tensor(mx["decay"], dtype=h.dtype))
    o = rms_norm(o.reshape(T, H * dv), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def retention_mixer(h: torch.Tensor, positions: torch.Tensor, w: Dict[str, torch.Tensor], mx: dict, eps: float) -> torch.Tensor:
    """Half-split rotation of q and k; k times dim^-1/2 after it; every head's output over its own root mean
    square (no weight); SiLU gate; output projection."""
    H, dk, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    T = h.shape[0]
    rot = mx["rot"]
    q = rotate((h @ w["q"].T).reshape(T, H, dk), positions, float(rot["base"]), int(rot["dims"]), "half")
    k = rotate((h @ w["k"].T).reshape(T, H, dk), positions, float(rot["base"]), int(rot["dims"]), "half") * dk ** -0.5
    v = (h @ w["v"].T).reshape(T, H, dv)
    o, _ = decayed_linear_attention(q, k, v, torch.tensor(mx["decay"], dtype=h.dtype))
    o = rms_norm(o, None, eps).reshape(T, H * dv) * silu(h @ w["g"].T)
    return o @ w["o"].T


# ------------------------------------------------------------------------------ routed feed-forward
def route_sigmoid(h: torch.Tensor, router: torch.Tensor, top: int):
    """-> (ids [T, top], weights [T, top]): the `top` largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ router.T)
    w, ids = torch.topk(s, top, dim=-1)
    return ids, w


def expert(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(x @ gate.T) * (x @ up.T)) @ down.T


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """sum over the chosen experts of expert(weight * h): the weight multiplies the expert's input."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    ids, wt = route_sigmoid(h, w["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(ids[t, j])
            assert e < E
            out[t] += expert(wt[t, j] * h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    return out


# ------------------------------------------------------------------------------ the model
def layer_runs(cfg: dict) -> List[tuple]:
    """Order in which the layers run: [(layer index, True when the embedding is added right before it)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(l, False) for l in range(a)]
    for p in range(times):
        runs += [(l, p > 0 and l == a) for l in range(a, b)]
    runs += [(l, False) for l in range(b, n)]
    return runs


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layer_outputs: Optional[list] = None):
    """Logits [T, vocab] of one sequence from position 0.  layer_outputs, if a list, receives the residual
    stream after every layer run."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.shape[0])
    e = W["embed"][tokens] * float(cfg["embedding"]["scale"])
    x = e.clone()
    for l, again in layer_runs(cfg):
        layer = cfg["layers"][l]
        if again:
            x = x + e
        h = rms_norm(x, W[f"l{l}.norm1"], eps)
        mw, mx = sub(W, f"l{l}.mix."), layer["mixer"]
        if layer["type"] == "attention":
            y = attention_mixer(h, pos, mw, mx, eps)
        elif layer["type"] == "retention":
            y = retention_mixer(h, pos, mw, mx, eps)
        elif layer["type"] == "lightning":
            y = lightning_mixer(h, mw, mx, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + moe_ff(h, sub(W, f"l{l}.mlp."), layer["mlp"])
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Checkpoint tensor names and shapes (linear weights are [out, in])."""
    D, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, tuple] = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for l, layer in enumerate(cfg["layers"]):
        p, mx = f"l{l}.", layer["mixer"]
        H, dk = int(mx["heads"]), int(mx["dim"])
        out[p + "norm1"] = (D,)
        if layer["type"] == "attention":
            out[p + "mix.q"], out[p + "mix.k"] = (H * dk, D), (int(mx["kv_heads"]) * dk, D)
            out[p + "mix.o"] = (D, H * dk)
        else:
            dv = int(mx["vdim"])
            out[p + "mix.q"] = out[p + "mix.k"] = (H * dk, D)
            out[p + "mix.v"] = out[p + "mix.g"] = (H * dv, D)
            out[p + "mix.o"] = (D, H * dv)
            if layer["type"] == "lightning":
                out[p + "mix.norm"] = (H * dv,)
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = int(mlp["expert"]["ff"])
            for e in range(int(mlp["router"]["experts"])):
                out[p + f"mlp.e{e}.gate"] = out[p + f"mlp.e{e}.up"] = (ff, D)
                out[p + f"mlp.e{e}.down"] = (D, ff)
            out[p + "mlp.router"] = (int(mlp["router"]["experts"]), D)
    return out


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with the design's tensor names: linear weights N(0, 1 / in), norm weights around 1,
    router rows large enough to spread the choice and the scores over (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(tuple(shape), generator=g)
        if name.endswith("norm") or name.endswith("norm1"):
            x = 1.0 + 0.2 * x
        elif name.endswith("mlp.router"):
            x = 2.0 * x / math.sqrt(shape[-1])
        elif name != "embed":
            x = x / math.sqrt(shape[-1])
        out[name] = x.to(torch.bfloat16)
    return out
