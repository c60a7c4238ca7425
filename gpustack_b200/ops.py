"""Operator wrappers: torch CUDA tensors in, libb200.so kernels on torch's current stream.

Each function mirrors one entry point of include/b200.h (and through it one operator of the
reference's vLLM backend).  torch is used for memory and streams only; there is deliberately no
eager/PyTorch fallback -- a missing library or a non-CUDA tensor raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .lib import B200Error, check, load

BLOCK_SIZE = 16  # tokens per KV page (vLLM default block_size)
# A/B switch: B200_LAYER_LIST_TC=0 keeps the layer-list families off the tensor cores (every product on the CUDA-core
# kernels, attention on the generic kernels) -- to tell a rounding effect from a fault of a tensor-core route
LAYER_LIST_TC = __import__("os").environ.get("B200_LAYER_LIST_TC", "1") != "0"


class KernelTimer:
    """Optional per-launch CUDA-event timing of the GEMM kernel (bench.py's live roofline).
    Events are recorded on the launching stream around each launch; nothing is recorded while a
    CUDA graph is being captured."""

    def __init__(self):
        self.records = []   # (tag, flops, bytes, start_event, end_event)

    def summary(self):
        torch.cuda.synchronize()
        agg = {}
        for tag, flops, nbytes, e0, e1 in self.records:
            a = agg.setdefault(tag, {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            a["launches"] += 1; a["ms"] += e0.elapsed_time(e1); a["flops"] += flops; a["bytes"] += nbytes
        return agg


TIMER: Optional[KernelTimer] = None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _req(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise B200Error(f"{name}: expected a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise B200Error(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise B200Error(f"{name}: tensor must be contiguous")


def device_info() -> dict:
    lib = load()
    v = [C.c_int() for _ in range(4)]
    check(lib.b200_device_info(*[C.byref(x) for x in v]), "device_info")
    return {"sm_count": v[0].value, "cc": (v[1].value, v[2].value), "l2_bytes": v[3].value}


# ------------------------------------------------------------------------------ normalisation
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None):
    _req(x, torch.bfloat16, "x"); _req(w, torch.bfloat16, "w")
    T, H = x.shape
    y = torch.empty_like(x) if out is None else out
    check(load().b200_rms_norm(_p(x), _p(w), _p(y), T, H, eps, _stream()), "rms_norm")
    return y


def fused_add_rms_norm(x, residual, w, eps, out=None, residual_out=None):
    """returns (y, residual_out); pass out=x, residual_out=residual for the in-place form."""
    _req(x, torch.bfloat16, "x"); _req(residual, torch.bfloat16, "residual"); _req(w, torch.bfloat16, "w")
    T, H = x.shape
    y = torch.empty_like(x) if out is None else out
    r = torch.empty_like(x) if residual_out is None else residual_out
    check(load().b200_fused_add_rms_norm(_p(x), _p(residual), _p(w), _p(y), _p(r), T, H, eps, _stream()),
          "fused_add_rms_norm")
    return y, r


def fused_add_rms_norm_partials(partials, residual, w, eps, out, residual_out):
    _req(partials, torch.float32, "partials"); _req(w, torch.bfloat16, "w")
    S, T, H = partials.shape
    check(load().b200_fused_add_rms_norm_partials(_p(partials), S, _p(residual), _p(w), _p(out),
                                                  _p(residual_out), T, H, eps, _stream()),
          "fused_add_rms_norm_partials")
    return out, residual_out


# ------------------------------------------------------------------- rope + kv-cache scatter
def rope_kv_write(qkv, positions, cos_sin, k_cache, v_cache, slot_mapping, Hq, Hkv, D):
    _req(qkv, torch.bfloat16, "qkv"); _req(positions, torch.int32, "positions")
    _req(cos_sin, torch.bfloat16, "cos_sin"); _req(slot_mapping, torch.int32, "slot_mapping")
    _req(k_cache, torch.bfloat16, "k_cache"); _req(v_cache, torch.bfloat16, "v_cache")
    T = qkv.shape[0]
    if qkv.shape[1] != (Hq + 2 * Hkv) * D:
        raise B200Error("rope_kv_write: qkv width mismatch")
    check(load().b200_rope_kv_write(_p(qkv), _p(positions), _p(cos_sin), _p(k_cache), _p(v_cache),
                                    _p(slot_mapping), T, Hq, Hkv, D, k_cache.shape[2], _stream()),
          "rope_kv_write")


def rope_kv_write_partials(partials, qkv_out, positions, cos_sin, k_cache, v_cache, slot_mapping, Hq, Hkv, D,
                           bias=None):
    """partials [S,T,(Hq+2Hkv)*D] fp32 (split-K QKV GEMM) -> rotated bf16 qkv_out + cache scatter."""
    _req(partials, torch.float32, "partials"); _req(qkv_out, torch.bfloat16, "qkv_out")
    S, T, W = partials.shape
    if W != (Hq + 2 * Hkv) * D or qkv_out.shape[1] != W:
        raise B200Error("rope_kv_write_partials: qkv width mismatch")
    check(load().b200_rope_kv_write_partials(_p(partials), S, _p(bias), _p(qkv_out), _p(positions), _p(cos_sin), _p(k_cache),
                                             _p(v_cache), _p(slot_mapping), T, Hq, Hkv, D, k_cache.shape[2],
                                             _stream()), "rope_kv_write_partials")


def silu_and_mul(x, out=None):
    _req(x, torch.bfloat16, "x")
    T, I2 = x.shape
    y = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device) if out is None else out
    check(load().b200_silu_and_mul(_p(x), _p(y), T, I2 // 2, _stream()), "silu_and_mul")
    return y


def embedding(ids, table, out=None, vocab_start=0, vocab_end=None):
    _req(ids, torch.int32, "ids"); _req(table, torch.bfloat16, "table")
    T, H = ids.shape[0], table.shape[1]
    y = torch.empty((T, H), dtype=table.dtype, device=table.device) if out is None else out
    ve = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    check(load().b200_embedding(_p(ids), _p(table), _p(y), T, H, vocab_start, ve, _stream()), "embedding")
    return y


def argmax(logits, out_idx=None, out_val=None):
    _req(logits, torch.float32, "logits")
    B, V = logits.shape
    idx = torch.empty((B,), dtype=torch.int32, device=logits.device) if out_idx is None else out_idx
    check(load().b200_argmax_f32(_p(logits), logits.stride(0), _p(idx), _p(out_val), B, V, _stream()),
          "argmax")
    return idx


def sample(logits, temps, seeds, out_idx=None, out_val=None, vocab_offset: int = 0):
    """Greedy (temps == 0) or Gumbel-max temperature sampling per row in ONE pass over the logits.
    temps: fp32 [B]; seeds: int32/uint32 [B] (bit patterns); returns int32 token ids (shard-local)."""
    _req(logits, torch.float32, "logits"); _req(temps, torch.float32, "temps"); _req(seeds, torch.int32, "seeds")
    B, V = logits.shape
    idx = torch.empty((B,), dtype=torch.int32, device=logits.device) if out_idx is None else out_idx
    check(load().b200_sample_f32(_p(logits), logits.stride(0), _p(temps), _p(seeds), vocab_offset, _p(idx), _p(out_val),
                                 B, V, _stream()), "sample")
    return idx


def gather_rows(x, rows, out=None):
    _req(x, torch.bfloat16, "x"); _req(rows, torch.int32, "rows")
    n, H = rows.shape[0], x.shape[1]
    y = torch.empty((n, H), dtype=x.dtype, device=x.device) if out is None else out
    check(load().b200_gather_rows(_p(x), _p(rows), _p(y), n, H, _stream()), "gather_rows")
    return y


# --------------------------------------------------------------------------------------- GEMM
def gemm_suggest_splits(M: int, N: int, K: int) -> int:
    return load().b200_gemm_suggest_splits(M, N, K)


def gemm(x, w, out=None, out_dtype=torch.bfloat16, splits: int = 1, block_x: int = 0):
    """y = x @ w.T (x [M,K], w [N,K], bf16).  splits>1 returns fp32 partials [splits, M, N]."""
    if not (x.is_cuda and w.is_cuda) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise B200Error("gemm: bf16 CUDA tensors required")
    if x.stride(-1) != 1 or w.stride(-1) != 1:
        raise B200Error("gemm: K must be the contiguous dimension")
    M, K = x.shape
    N = w.shape[0]
    out_f32 = 1 if (out_dtype == torch.float32 or splits > 1) else 0
    if out is None:
        shape = (splits, M, N) if splits > 1 else (M, N)
        out = torch.empty(shape, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    ldy = out.stride(-2)
    timed = TIMER is not None and not torch.cuda.is_current_stream_capturing()
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(load().b200_gemm_bf16_ex(_p(x), _p(w), _p(out), M, N, K, x.stride(0), w.stride(0), ldy, out_f32,
                                   splits, block_x, _stream()), "gemm")
    if timed:
        e1.record()
        tag = "gemm_prefill" if M > 256 else "gemm_decode"
        TIMER.records.append((tag, 2.0 * M * N * K, 2.0 * (N * K + M * K) + (4.0 if out_f32 else 2.0) * M * N * splits,
                              e0, e1))
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I,H] gate and up weights -> [2I,H] with row 2i = gate_i, row 2i+1 = up_i (the layout
    gemm_silu_mul expects)."""
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()


def gemm_silu_mul(x, w_interleaved, out=None):
    """act = silu(x @ gate.T) * (x @ up.T) in one kernel; w_interleaved from interleave_gate_up."""
    if not (x.is_cuda and w_interleaved.is_cuda) or x.dtype != torch.bfloat16 or w_interleaved.dtype != torch.bfloat16:
        raise B200Error("gemm_silu_mul: bf16 CUDA tensors required")
    M, K = x.shape
    N = w_interleaved.shape[0]
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    timed = TIMER is not None and not torch.cuda.is_current_stream_capturing()
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    check(load().b200_gemm_bf16_silu_mul(_p(x), _p(w_interleaved), _p(out), M, N, K, x.stride(0),
                                         w_interleaved.stride(0), out.stride(0), _stream()), "gemm_silu_mul")
    if timed:
        e1.record()
        TIMER.records.append(("gemm_prefill" if M > 256 else "gemm_decode", 2.0 * M * N * K,
                              2.0 * (N * K + M * K) + 1.0 * M * N, e0, e1))
    return out


# --------------------------------------------------------------------------------------- fp8 (W8A8)
FP8 = torch.float8_e4m3fn


def quant_fp8_per_token(x, out=None, scales=None):
    """Dynamic per-token e4m3 quantisation: returns (q [T,K] float8_e4m3fn, scales [T] fp32)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise B200Error("quant_fp8_per_token: bf16 CUDA tensor with contiguous rows required")
    T, K = x.shape
    q = torch.empty((T, K), dtype=FP8, device=x.device) if out is None else out
    sc = torch.empty((T,), dtype=torch.float32, device=x.device) if scales is None else scales
    check(load().b200_quant_fp8_per_token(_p(x), x.stride(0), _p(q), q.stride(0), _p(sc), T, K, _stream()),
          "quant_fp8_per_token")
    return q, sc


def gemm_fp8(xq, xscale, wq, wscale, out=None, out_dtype=torch.bfloat16, splits: int = 1, silu_mul: bool = False):
    """y = (xq @ wq.T) * xscale[:,None] * wscale  (e4m3 operands, fp32 accumulate).  wscale: fp32
    tensor with 1 element (per-tensor) or N elements (per output channel).  silu_mul: wq holds
    interleaved gate/up rows and y = silu(gate) * up, [M, N/2] bf16."""
    if not (xq.is_cuda and wq.is_cuda) or xq.dtype != FP8 or wq.dtype != FP8:
        raise B200Error("gemm_fp8: float8_e4m3fn CUDA tensors required (there is no CPU path)")
    if xq.stride(-1) != 1 or wq.stride(-1) != 1:
        raise B200Error("gemm_fp8: K must be the contiguous dimension")
    _req(xscale, torch.float32, "xscale"); _req(wscale, torch.float32, "wscale")
    M, K = xq.shape
    N = wq.shape[0]
    if xscale.numel() != M or wscale.numel() not in (1, N):
        raise B200Error("gemm_fp8: xscale must have M elements, wscale 1 or N")
    out_f32 = 1 if (out_dtype == torch.float32 or splits > 1) else 0
    if out is None:
        shape = (splits, M, N) if splits > 1 else (M, N // 2 if silu_mul else N)
        out = torch.empty(shape, dtype=torch.float32 if out_f32 else torch.bfloat16, device=xq.device)
    check(load().b200_gemm_fp8(_p(xq), _p(wq), _p(out), M, N, K, xq.stride(0), wq.stride(0), out.stride(-2),
                               _p(xscale), _p(wscale), 0 if wscale.numel() == 1 else 1, out_f32, splits,
                               1 if silu_mul else 0, _stream()), "gemm_fp8")
    return out


# --------------------------------------------------------------------------------------- MoE
ROUTER_PAD = 128   # the router weight is zero-padded to one full weight tile of the GEMM


def pad_router(router: torch.Tensor) -> torch.Tensor:
    """[E, H] -> [128, H] with zero rows, so the router projection is an ordinary one-tile GEMM."""
    out = torch.zeros(ROUTER_PAD, router.shape[1], dtype=router.dtype, device=router.device)
    out[: router.shape[0]] = router
    return out


def moe_block_x(n_pairs: int, num_experts: int) -> int:
    """Row-tile width of the permuted MoE row space: about the mean rows per expert, so that the
    padding (< block_x rows per expert) stays a small fraction of the grouped GEMMs."""
    avg = n_pairs / max(1, num_experts)
    for bx in (256, 128, 64):
        if avg >= 0.75 * bx:
            return bx
    return 32


def moe_capacity_rows(n_pairs: int, num_experts: int, block_x: int) -> int:
    return load().b200_moe_capacity_rows(n_pairs, num_experts, block_x)


class MoEWorkspace:
    """Device buffers of one MoE dispatch (sized for `max_tokens` tokens, reused by every layer)."""

    def __init__(self, max_tokens: int, top_k: int, num_experts: int, H: int, I: int, device):
        self.top_k, self.E, self.H, self.I = top_k, num_experts, H, I
        n_pairs = max_tokens * top_k
        cap = max(moe_capacity_rows(n_pairs, num_experts, bx) for bx in (32, 64, 128, 256))
        i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=device)   # noqa: E731
        self.capacity = cap
        self.logits = torch.empty(max_tokens, ROUTER_PAD, dtype=torch.bfloat16, device=device)
        self.topk_ids, self.topk_w = i32(n_pairs), torch.empty(n_pairs, dtype=torch.float32, device=device)
        self.pair_row, self.row_pair = i32(n_pairs), i32(cap)
        self.row_weight = torch.empty(cap, dtype=torch.float32, device=device)
        self.tile_expert, self.num_tiles = i32(cap // 32 + 1), torch.zeros(2, dtype=torch.int32, device=device)
        self.xp = torch.empty(cap, H, dtype=torch.bfloat16, device=device)
        self.act = torch.empty(cap, I, dtype=torch.bfloat16, device=device)
        self.yp = torch.empty(cap, H, dtype=torch.bfloat16, device=device)


def moe_route(router_logits, top_k: int, renormalize: bool = True, out_ids=None, out_w=None,
              num_experts: Optional[int] = None):
    """router_logits [T, >=E] bf16 (columns beyond num_experts are padding of the router GEMM)."""
    if not router_logits.is_cuda or router_logits.dtype != torch.bfloat16 or router_logits.stride(1) != 1:
        raise B200Error("moe_route: bf16 CUDA logits with contiguous rows required")
    T = router_logits.shape[0]
    E = router_logits.shape[1] if num_experts is None else num_experts
    ids = torch.empty(T * top_k, dtype=torch.int32, device=router_logits.device) if out_ids is None else out_ids
    w = torch.empty(T * top_k, dtype=torch.float32, device=router_logits.device) if out_w is None else out_w
    check(load().b200_moe_route(_p(router_logits), router_logits.stride(0), _p(ids), _p(w), T, E, top_k,
                                1 if renormalize else 0, _stream()), "moe_route")
    return ids, w


def moe_experts(x, router_logits, w13, w2, top_k: int, ws: MoEWorkspace, out, renormalize: bool = True):
    """out[t] = sum_k weight_k * down_k(silu(gate_k x) * up_k x) over the top-k experts of token t.
    x [T,H] bf16; router_logits [T,>=E] bf16; w13 [E*2I, H] (per expert: interleaved gate/up rows);
    w2 [E*H, I].  Seven launches: route, align, gather, grouped gate_up+SiLU, grouped down (x routing
    weight), combine -- no host synchronisation."""
    T, H = x.shape
    E, I = ws.E, ws.I
    n_pairs = T * top_k
    bx = moe_block_x(n_pairs, E)
    cap = moe_capacity_rows(n_pairs, E, bx)
    if cap > ws.capacity:
        raise B200Error(f"moe_experts: {T} tokens exceed the workspace ({ws.capacity} rows)")
    L, st = load(), _stream()
    moe_route(router_logits, top_k, renormalize, out_ids=ws.topk_ids, out_w=ws.topk_w, num_experts=E)
    check(L.b200_moe_align(_p(ws.topk_ids), _p(ws.topk_w), n_pairs, E, bx, cap, _p(ws.pair_row), _p(ws.row_pair),
                           _p(ws.row_weight), _p(ws.tile_expert), _p(ws.num_tiles), st), "moe_align")
    check(L.b200_moe_gather(_p(x), _p(ws.row_pair), _p(ws.num_tiles), _p(ws.xp), H, top_k, cap, st), "moe_gather")
    check(L.b200_moe_grouped_gemm(_p(ws.xp), _p(w13), _p(ws.act), cap, 2 * I, H, E, H, w13.stride(0), I, None,
                                  _p(ws.tile_expert), _p(ws.num_tiles), bx, 1, st), "moe_grouped_gemm(gate_up)")
    check(L.b200_moe_grouped_gemm(_p(ws.act), _p(w2), _p(ws.yp), cap, H, I, E, I, w2.stride(0), H, _p(ws.row_weight),
                                  _p(ws.tile_expert), _p(ws.num_tiles), bx, 0, st), "moe_grouped_gemm(down)")
    check(L.b200_moe_combine(_p(ws.yp), _p(ws.pair_row), _p(out), T, H, top_k, st), "moe_combine")
    return out


MOE_LAUNCHES = 6


def splitk_reduce(partials, out=None):
    _req(partials, torch.float32, "partials")
    S, M, N = partials.shape
    y = torch.empty((M, N), dtype=torch.bfloat16, device=partials.device) if out is None else out
    check(load().b200_splitk_reduce(_p(partials), S, _p(y), M, N, y.stride(0), _stream()), "splitk_reduce")
    return y


# ---------------------------------------------------------------------------------- attention
def attn_decode_splits(B, Hkv, max_seq_len) -> int:
    return load().b200_attn_decode_splits(B, Hkv, max_seq_len, BLOCK_SIZE)


def attn_decode_workspace(B, Hq, D, num_splits, device) -> torch.Tensor:
    n = load().b200_attn_decode_workspace_bytes(B, Hq, D, num_splits)
    # zeroed ONCE: the first bytes hold the per-(sequence, kv-head) arrival counters of the in-kernel
    # split merge, which reset themselves after every launch
    return torch.zeros((n + 3) // 4, dtype=torch.float32, device=device)


def paged_attn_decode(q, q_stride, k_cache, v_cache, block_table, seq_lens, out, Hq, Hkv, D, scale,
                      num_splits=1, workspace=None, sink=None, gate=None, window: int = 0, gate_per_head: bool = False,
                      lse_out=None):
    """q: [B, >=Hq*D] view into the qkv buffer (row stride q_stride elements).  sink [Hq] fp32: softmax sink;
    gate [B, >=Hq*D] bf16 view (same row stride rule): the output is multiplied by sigmoid(gate) -- with gate_per_head
    the view holds ONE number per head, [B, >=Hq]; window > 0: the row at position n - 1 sees keys [n - window, n)."""
    B = seq_lens.shape[0]
    _req(block_table, torch.int32, "block_table"); _req(seq_lens, torch.int32, "seq_lens")
    if lse_out is not None:       # fp32 [B, Hq]: every row's log-sum-exp, for attn_sink_decode_more
        _req(lse_out, torch.float32, "lse_out")
    check(load().b200_paged_attn_decode_lse(_p(q), q_stride, _p(k_cache), _p(v_cache), _p(block_table),
                                            block_table.shape[1], _p(seq_lens), _p(out), _p(workspace),
                                            num_splits, B, Hq, Hkv, D, k_cache.shape[2], scale, _p(sink), _p(gate),
                                            0 if gate is None else gate.stride(0), int(window), 1 if gate_per_head else 0,
                                            _p(lse_out), _stream()), "paged_attn_decode")
    return out


def attn_prefill_tile(Hq, Hkv) -> int:
    t = load().b200_attn_prefill_tile(Hq, Hkv)
    if t <= 0:
        raise B200Error(f"prefill attention: unsupported head grouping {Hq}/{Hkv}")
    return t


def build_prefill_tiles(q_lens: Sequence[int], tile: int, ctx_lens: Optional[Sequence[int]] = None):
    """Host-side tile list for b200_paged_attn_prefill: (tile_seq, tile_q0) int32 lists, ordered
    heaviest first (a causal tile's work grows with its last key position), so the long tiles do
    not end up alone in the last wave."""
    tiles = []
    for s, n in enumerate(q_lens):
        c = 0 if ctx_lens is None else int(ctx_lens[s])
        for q0 in range(0, n, tile):
            tiles.append((c + q0 + tile, s, q0))
    tiles.sort(key=lambda t: -t[0])
    return [t[1] for t in tiles], [t[2] for t in tiles]


def attn_prefill_tc_covers(Hq, Hkv, D) -> bool:
    return bool(load().b200_attn_prefill_tc_covers(Hq, Hkv, D))


def paged_attn_prefill_ex(q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, out, Hq, Hkv, D,
                          scale, sink=None, gate=None, window: int = 0, gate_per_head: bool = False, lse_out=None):
    """The tcgen05 prefill kernel with a softmax sink ([Hq] fp32), a sigmoid output gate (bf16 view [T, >=Hq*D], or
    [T, >=Hq] with gate_per_head: one number per head) and / or a sliding window (position i sees j with
    0 <= i - j < window); only for shapes attn_prefill_tc_covers() accepts, tiles of attn_prefill_tile(Hq, Hkv) rows."""
    if lse_out is not None:       # fp32 [T, Hq]: every row's log-sum-exp, for attn_sink_prefill_more
        _req(lse_out, torch.float32, "lse_out")
    check(load().b200_paged_attn_prefill_lse(_p(q), q_stride, q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0],
                                             _p(block_table), block_table.shape[1], _p(cu_q), _p(ctx_lens), _p(tile_seq),
                                             _p(tile_q0), tile_seq.shape[0], _p(out), Hq, Hkv, D, k_cache.shape[2], scale,
                                             _p(sink), _p(gate), 0 if gate is None else gate.stride(0), int(window),
                                             1 if gate_per_head else 0, _p(lse_out), _stream()), "paged_attn_prefill_ex")
    return out


def paged_attn_prefill(q, q_stride, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0,
                       out, Hq, Hkv, D, scale):
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (ctx_lens, "ctx_lens"),
                 (tile_seq, "tile_seq"), (tile_q0, "tile_q0")):
        _req(t, torch.int32, n)
    check(load().b200_paged_attn_prefill(_p(q), q_stride, q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0],
                                         _p(block_table), block_table.shape[1], _p(cu_q), _p(ctx_lens), _p(tile_seq),
                                         _p(tile_q0), tile_seq.shape[0], _p(out), Hq, Hkv, D,
                                         k_cache.shape[2], scale, _stream()), "paged_attn_prefill")
    return out


# ----------------------------------------------------------- layer-list decoders (fp32 residual stream)
def _is_f32(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 1
    if t.dtype == torch.bfloat16:
        return 0
    raise B200Error(f"expected bf16 or fp32, got {t.dtype}")


def _cuda(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise B200Error("expected CUDA tensors (there is no CPU path)")


def linear(x, w, out, bias=None, relu2: bool = False, force_simt: bool = False):
    """out = x @ w.T (+ bias); relu2: out = max(., 0)^2 (in the GEMM's epilogue on the tensor-core path).  bf16 x / bf16 or fp32 out with K a multiple of 64 and 16-byte aligned rows
    go to the tcgen05 GEMM; every other case (fp32 activations = a model served in true 32-bit; odd
    shapes) runs on the CUDA cores with fp32 FMA accumulation."""
    _cuda(x, w, out, bias)
    if w.dtype != torch.bfloat16 or x.stride(-1) != 1 or w.stride(-1) != 1 or out.stride(-1) != 1:
        raise B200Error("linear: bf16 weights and contiguous rows required")
    M, K = x.shape
    N = w.shape[0]
    xf, yf = _is_f32(x), _is_f32(out)
    if (LAYER_LIST_TC and not force_simt and not xf and bias is None and K % 64 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and (out.stride(0) * out.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        if not relu2:
            return gemm(x, w, out=out, out_dtype=out.dtype)
        if not yf:
            timed = TIMER is not None and not torch.cuda.is_current_stream_capturing()
            if timed:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            check(load().b200_gemm_bf16_relu2(_p(x), _p(w), _p(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                                              _stream()), "gemm_relu2")
            if timed:
                e1.record()
                TIMER.records.append(("gemm_prefill" if M > 256 else "gemm_decode", 2.0 * M * N * K,
                                      2.0 * (N * K + M * K) + 2.0 * M * N, e0, e1))
            return out
        gemm(x, w, out=out, out_dtype=out.dtype)
        return relu2_(out)
    check(load().b200_linear_simt(_p(x), xf, _p(w), _p(bias), _p(out), yf, M, N, K, x.stride(0), w.stride(0),
                                  out.stride(0), _stream()), "linear_simt")
    return relu2_(out) if relu2 else out


def sum_layer_norm(y, x_in, w, alpha: float, eps: float, x_out=None, xb_out=None, rows=None, out_scale: float = 1.0):
    """o = LN(alpha * x_in + y) * w * out_scale (y None: LN(x_in); rows: gather x_in[rows]); fp32 statistics.
    x_out (fp32 residual stream) and / or xb_out (next projection's input, bf16 or fp32) receive o."""
    _cuda(y, x_in, w, x_out, xb_out, rows)
    if x_in.dtype != torch.float32 or (x_out is not None and x_out.dtype != torch.float32):
        raise B200Error("sum_layer_norm: the residual stream is fp32")
    D = x_in.shape[1]
    T = (rows.shape[0] if rows is not None else x_in.shape[0]) if y is None else y.shape[0]
    check(load().b200_sum_layer_norm(_p(y), 0 if y is None else _is_f32(y), 0 if y is None else y.stride(0), _p(x_in),
                                     _p(rows), _p(w), _p(x_out), _p(xb_out), 0 if xb_out is None else _is_f32(xb_out),
                                     T, D, alpha, eps, out_scale, _stream()), "sum_layer_norm")


def embed_rows(ids, table, x_out, xb_out=None):
    _cuda(ids, table, x_out, xb_out)
    _req(ids, torch.int32, "ids"); _req(table, torch.bfloat16, "table"); _req(x_out, torch.float32, "x_out")
    check(load().b200_embed_rows_f32(_p(ids), _p(table), _p(x_out), _p(xb_out), 0 if xb_out is None else _is_f32(xb_out),
                                     ids.shape[0], table.shape[1], table.shape[0], _stream()), "embed_rows")


def relu2_(u):
    return relu2(u)


def relu2(u, out=None):
    _cuda(u, out)
    out = u if out is None else out
    if not u.is_contiguous() or not out.is_contiguous():
        raise B200Error("relu2: contiguous tensors required")
    check(load().b200_relu2(_p(u), _p(out), _is_f32(u), u.numel(), _stream()), "relu2")
    return out


def attn_prep(proj, bias, q_norm, k_norm, positions, slots, k_cache, v_cache, H, G, dk, dv, eps,
              temp_coef: float = 0.0, temp_every: int = 0):
    """In place on the fused projection rows: bias, per-head RMS norm of q and k, query temperature; k and v
    go to their pages (k_cache None: a mixer that reads another layer's cache)."""
    _cuda(proj, bias, q_norm, k_norm, positions, slots, k_cache, v_cache)
    has_kv = k_cache is not None
    page = k_cache.shape[2] if has_kv else 1
    check(load().b200_attn_prep(_p(proj), _is_f32(proj), proj.stride(0), _p(bias), _p(q_norm), _p(k_norm), _p(positions),
                                _p(slots), _p(k_cache), _p(v_cache), proj.shape[0], H, G, dk, dv, page, 1 if has_kv else 0,
                                eps, temp_coef, temp_every, _stream()), "attn_prep")


def attn_sink_prefill_tile() -> int:
    return load().b200_attn_sink_prefill_tile()


def _pool_args(pool, k_cache, dk, dv):
    """pool = (pool_k, pool_v, block size) or None -> (pool_k ptr, pool_v ptr, block size, entries per page)."""
    if pool is None:
        return None, None, 0, 0
    pk, pv, n = pool
    _cuda(pk, pv)
    _req(pk, torch.float32, "pool_k"); _req(pv, torch.float32, "pool_v")
    per_page = -(-k_cache.shape[2] // n)
    if pk.shape[2] != per_page or pk.shape[3] != dk or pv.shape[3] != dv:
        raise B200Error("pooled cache: [blocks, G, ceil(page / pool), width] expected")
    return _p(pk), _p(pv), int(n), per_page


def attn_sink_prefill(proj, gate_col, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, sink, out,
                      H, G, dk, dv, scale, tile_rows: int = 0, v_ld: int = 0, window: int = 0, gate_per_head: bool = False,
                      head_scale=None, pool=None):
    """v_ld: elements between value rows (0 = dv); v_cache is k_cache and v_ld == dk when the values are the
    first dv entries of the key rows (a latent cache).  window > 0: position i sees j with 0 <= i - j < window.
    gate_per_head: the gate is ONE column per head at gate_col; head_scale: fp32 [H] factors on the score;
    pool = (pool_k, pool_v, n): beside the window, the mean key / value of every block of n tokens that ends at or
    before i - window (fp32 caches written by kv_pool_update)."""
    _cuda(proj, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, sink, out, head_scale)
    if k_cache.dtype != proj.dtype or out.dtype != proj.dtype:
        raise B200Error("attn_sink_prefill: projection, cache and output must share one element type")
    pk, pv, pn, ppp = _pool_args(pool, k_cache, dk, dv)
    check(load().b200_attn_sink_prefill_pool(_p(proj), _is_f32(proj), proj.stride(0), gate_col, _p(k_cache), _p(v_cache),
                                             _p(block_table), block_table.shape[1], _p(cu_q), _p(ctx_lens), _p(tile_seq),
                                             _p(tile_q0), tile_seq.shape[0], tile_rows or attn_sink_prefill_tile(), _p(sink),
                                             _p(out), out.stride(0), H, G, dk, dv, k_cache.shape[2], scale, v_ld, int(window),
                                             1 if gate_per_head else 0, _p(head_scale), pk, pv, pn, ppp, _stream()),
          "attn_sink_prefill")
    return out


def attn_sink_prefill_more(proj, k_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, out, init_lse, H, G, dk, dv, scale,
                           tile_rows: int, window: int, head_scale, pool):
    """Continues a softmax over the pooled blocks: `out` holds the normalised attention over the window's tokens (another
    kernel's), init_lse [T, H] its log-sum-exp; `out` is rewritten with the joint result.  head_scale multiplies `scale`
    here only: the first part must have been run with the same per-head scale."""
    _cuda(proj, k_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, out, init_lse, head_scale)
    _req(init_lse, torch.float32, "init_lse")
    pk, pv, pn, ppp = _pool_args(pool, k_cache, dk, dv)
    check(load().b200_attn_sink_prefill_more(_p(proj), _is_f32(proj), proj.stride(0), _p(k_cache), _p(block_table),
                                             block_table.shape[1], _p(cu_q), _p(ctx_lens), _p(tile_seq), _p(tile_q0),
                                             tile_seq.shape[0], tile_rows, _p(out), out.stride(0), H, G, dk, dv,
                                             k_cache.shape[2], scale, int(window), _p(head_scale), pk, pv, pn, ppp, _p(init_lse),
                                             _stream()), "attn_sink_prefill_more")
    return out


def attn_sink_decode_more(proj, k_cache, block_table, seq_lens, out, init_lse, H, G, dk, dv, scale, window: int, head_scale,
                          pool):
    """Single rows: continues a softmax over the pooled blocks.  `out` holds the normalised attention over the window's
    tokens (another kernel's), init_lse [B, H] its log-sum-exp; `out` is rewritten with the joint result."""
    _cuda(proj, block_table, seq_lens, out, init_lse, head_scale)
    _req(init_lse, torch.float32, "init_lse")
    pk, pv, pn, ppp = _pool_args(pool, k_cache, dk, dv)
    check(load().b200_attn_sink_decode_more(_p(proj), _is_f32(proj), proj.stride(0), _p(block_table), block_table.shape[1],
                                            _p(seq_lens), seq_lens.shape[0], _p(out), out.stride(0), H, G, dk, dv,
                                            k_cache.shape[2], scale, int(window), _p(head_scale), pk, pv, pn, ppp, _p(init_lse),
                                            _stream()), "attn_sink_decode_more")
    return out


def attn_sink_decode(proj, gate_col, k_cache, v_cache, block_table, seq_lens, sink, out, H, G, dk, dv, scale,
                     v_ld: int = 0, window: int = 0, gate_per_head: bool = False, head_scale=None, pool=None):
    _cuda(proj, k_cache, v_cache, block_table, seq_lens, sink, out, head_scale)
    if k_cache.dtype != proj.dtype or out.dtype != proj.dtype:
        raise B200Error("attn_sink_decode: projection, cache and output must share one element type")
    pk, pv, pn, ppp = _pool_args(pool, k_cache, dk, dv)
    check(load().b200_attn_sink_decode_pool(_p(proj), _is_f32(proj), proj.stride(0), gate_col, _p(k_cache), _p(v_cache),
                                            _p(block_table), block_table.shape[1], _p(seq_lens), seq_lens.shape[0], _p(sink),
                                            _p(out), out.stride(0), H, G, dk, dv, k_cache.shape[2], scale, v_ld, int(window),
                                            1 if gate_per_head else 0, _p(head_scale), pk, pv, pn, ppp, _stream()),
          "attn_sink_decode")
    return out


def mlstm_state_slices(dv: int) -> int:
    return (dv + 31) // 32


def mlstm_scan(proj, q_col, k_col, v_col, gates, gate_bias, cu_seq, ctx_lens, state_slots, S, n, m, o_raw, H, dk, dv,
               cap: float, max_len: int = 1):
    """Runs every sequence's new rows through the matrix-memory recurrence (state slot in, state slot out).
    max_len: an upper bound of the new rows per sequence (prompt portions run in the chunk form)."""
    _cuda(proj, gates, gate_bias, cu_seq, ctx_lens, state_slots, S, n, m, o_raw)
    _req(gates, torch.float32, "gates"); _req(S, torch.float32, "S"); _req(o_raw, torch.float32, "o_raw")
    check(load().b200_mlstm_scan(_p(proj), _is_f32(proj), proj.stride(0), q_col, k_col, v_col, _p(gates), _p(gate_bias),
                                 _p(cu_seq), _p(ctx_lens), _p(state_slots), _p(S), _p(n), _p(m), _p(o_raw),
                                 state_slots.shape[0], H, dk, dv, cap, dk ** -0.5, int(max_len), _stream()), "mlstm_scan")


def mlstm_out(o_raw, proj, gate_col, norm_w, out, H, dv, eps):
    _cuda(o_raw, proj, norm_w, out)
    check(load().b200_mlstm_out(_p(o_raw), _p(proj), _is_f32(proj), proj.stride(0), gate_col, _p(norm_w), _p(out),
                                out.stride(0), o_raw.shape[0], H, dv, eps, _stream()), "mlstm_out")
    return out


# ------------------------------------------- pre-norm fp32 residual, rotation prep, decayed linear attention
def add_rms_norm(x_in, w, eps: float, a=None, b=None, c=None, x_out=None, xb_out=None, rows=None):
    """z = x_in + a + b + c (fp32 rows, addends optional); x_out = z; xb_out = RMSnorm(z) * w (bf16 or fp32).
    rows: gather -- row r reads source row rows[r] and only xb_out is written.  w None: the sum alone."""
    _cuda(x_in, a, b, c, w, x_out, xb_out, rows)
    for t_, n_ in ((x_in, "x_in"), (a, "a"), (b, "b"), (c, "c"), (x_out, "x_out")):
        if t_ is not None:
            _req(t_, torch.float32, n_)
    D = x_in.shape[1]
    T = rows.shape[0] if rows is not None else (xb_out if xb_out is not None else x_out).shape[0]
    check(load().b200_add_rms_norm_f32(_p(x_in), _p(a), _p(b), _p(c), _p(rows), _p(w), _p(x_out), _p(xb_out),
                                       0 if xb_out is None else _is_f32(xb_out), T, D, eps, _stream()), "add_rms_norm")


def rot_prep(proj, q_col: int, k_col: int, v_col: int, positions, slots, q_out, k_out, v_out, H, G, dk, dv, *,
             paged: bool, feature: Optional[str] = None, rot_dims: int = 0, half_layout: bool = False, freq=None,
             unit_norm: bool = False, eps: float = 0.0, q_mul: float = 1.0, k_mul: float = 1.0, q_head_mul=None):
    """Per-head feature map / rotation / unit norm / factor of a fused projection's q, k (and v) heads
    (csrc/rot_prep.cu).  paged: k_out / v_out are cache pages [blocks, G, page, width] written at slots[t]; otherwise
    row buffers.  v_col < 0: the values are the keys as projected.  q_head_mul: fp32 [H], one more factor per query head."""
    _cuda(proj, positions, slots, q_out, k_out, v_out, freq)
    if freq is not None:
        _req(freq, torch.float64, "freq")
    dst = q_out if q_out is not None else k_out
    if any(t_ is not None and t_.dtype != dst.dtype for t_ in (q_out, k_out, v_out)):
        raise B200Error("rot_prep: one destination element type")
    if k_out is None:          # a mixer that reads another layer's keys and values: queries only
        paged, v_out = False, None
    page = k_out.shape[2] if paged else 0
    _cuda(q_head_mul)
    check(load().b200_rot_prep_hm(_p(proj), _is_f32(proj), proj.stride(0), q_col, k_col, v_col, _p(positions), _p(slots),
                               _p(q_out), q_out.stride(0), _p(k_out), 0 if (paged or k_out is None) else k_out.stride(0), _p(v_out),
                               0 if (paged or v_out is None) else v_out.stride(0), _is_f32(dst), 1 if paged else 0, page,
                               proj.shape[0], H, G, dk, dv, {None: 0, "silu": 1}[feature], rot_dims, 1 if half_layout else 0,
                               _p(freq), 1 if unit_norm else 0, eps, q_mul, k_mul, _p(q_head_mul), _stream()), "rot_prep")


def linattn_scan(x, q_col: int, k_col: int, v_col: int, decay, cu_seq, ctx_lens, state_slots, S, o_raw, H, dk, dv,
                 max_len: int = 1):
    """Decayed linear attention over every sequence's new rows of the fp32 rows x (state slot in, state slot out).
    max_len: an upper bound of the new rows per sequence (prompt portions run in the chunk form)."""
    _cuda(x, decay, cu_seq, ctx_lens, state_slots, S, o_raw)
    _req(x, torch.float32, "x"); _req(S, torch.float32, "S"); _req(o_raw, torch.float32, "o_raw")
    _req(decay, torch.float32, "decay")
    check(load().b200_linattn_scan(_p(x), x.stride(0), q_col, k_col, v_col, _p(decay), _p(cu_seq), _p(ctx_lens),
                                   _p(state_slots), _p(S), _p(o_raw), state_slots.shape[0], H, dk, dv, int(max_len),
                                   _stream()), "linattn_scan")


def linattn_out(o_raw, proj, gate_col: int, norm_w, out, H, dv, eps: float, all_heads: bool, gate_act: str):
    _cuda(o_raw, proj, norm_w, out)
    check(load().b200_linattn_out(_p(o_raw), _p(proj), _is_f32(proj), proj.stride(0), gate_col, _p(norm_w), _p(out),
                                  out.stride(0), o_raw.shape[0], H, dv, 1 if all_heads else 0,
                                  {"sigmoid": 0, "silu": 1}[gate_act], eps, _stream()), "linattn_out")
    return out


# ------------------------------------------- norm before and after every sublayer, short convolutions, pooled KV blocks
def embed_pos(ids, positions, table, pos_table, x_out):
    """x_out[t] (fp32) = table[ids[t]] + pos_table[positions[t]]."""
    _cuda(ids, positions, table, pos_table, x_out)
    _req(ids, torch.int32, "ids"); _req(positions, torch.int32, "positions"); _req(table, torch.bfloat16, "table")
    _req(pos_table, torch.bfloat16, "pos_table"); _req(x_out, torch.float32, "x_out")
    check(load().b200_embed_pos_f32(_p(ids), _p(positions), _p(table), _p(pos_table), _p(x_out), ids.shape[0], table.shape[1],
                                    table.shape[0], pos_table.shape[0], _stream()), "embed_pos")


def sandwich_join(x_in, eps: float, y=None, y2=None, ya: float = 1.0, yb: float = 1.0, post_w=None, mult: float = 1.0,
                  pre_w=None, x_out=None, h_out=None, rows=None, zero_centred: bool = True):
    """z = x_in + mult * norm(ya * y + yb * y2; post_w) (y None: z = x_in); x_out = z; h_out = norm(z; pre_w) in fp32 or
    bf16.  norm(v; w) = v / sqrt(mean(v^2) + eps) * (1 + w) (zero_centred) or * w.  rows: gather, h_out only."""
    _cuda(x_in, y, y2, post_w, pre_w, x_out, h_out, rows)
    for t_, n_ in ((x_in, "x_in"), (y, "y"), (y2, "y2"), (x_out, "x_out")):
        if t_ is not None:
            _req(t_, torch.float32, n_)
    D = x_in.shape[1]
    T = rows.shape[0] if rows is not None else (h_out if h_out is not None else x_out).shape[0]
    check(load().b200_sandwich_join(_p(x_in), _p(y), _p(y2), ya, yb, _p(post_w), mult, _p(rows), _p(pre_w), _p(x_out), _p(h_out),
                                    0 if h_out is None else _is_f32(h_out), T, D, eps, 1 if zero_centred else 0, _stream()),
          "sandwich_join")


def causal_conv(x, w, ring, cu_seq, ctx_lens, state_slots, out, *, add_input: bool, in_bias=None, bias=None):
    """Causal per-channel convolution over every sequence's new rows (csrc/sandwich.cu).  x [T, C] (a column slice of
    wider rows is fine), w fp32 [C, taps] (last tap = current token), ring fp32 [slots, taps - 1, C]."""
    _cuda(x, w, ring, cu_seq, ctx_lens, state_slots, out, in_bias, bias)
    _req(w, torch.float32, "w")
    T, Cn = x.shape
    taps = w.shape[1]
    if x.stride(1) != 1 or out.stride(1) != 1 or (ring is not None and tuple(ring.shape[1:]) != (taps - 1, Cn)):
        raise B200Error("causal_conv: contiguous rows and a ring of [slots, taps - 1, channels]")
    check(load().b200_causal_conv(_p(x), _is_f32(x), x.stride(0), _p(in_bias), _p(w), _p(bias), 1 if add_input else 0, _p(ring),
                                  _p(cu_seq), _p(ctx_lens), _p(state_slots), state_slots.shape[0], _p(out), _is_f32(out),
                                  out.stride(0), T, Cn, taps, _stream()), "causal_conv")
    return out


def conv_commit(x, ring, cu_seq, ctx_lens, state_slots, taps: int, in_bias=None):
    """The last taps - 1 inputs of every sequence's new rows go to its ring; run after causal_conv."""
    _cuda(x, ring, cu_seq, ctx_lens, state_slots, in_bias)
    check(load().b200_conv_commit(_p(x), _is_f32(x), x.stride(0), _p(in_bias), _p(ring), _p(cu_seq), _p(ctx_lens),
                                  _p(state_slots), state_slots.shape[0], x.shape[1], taps, _stream()), "conv_commit")


def kv_pool_update(k_cache, v_cache, pool_k, pool_v, block_table, cu_q, ctx_lens, n_seqs: int, max_new: int, pool: int):
    """Mean key / value of the blocks of `pool` tokens completed by this step's rows.  cu_q None: one new row per
    sequence, ctx_lens counts it (a decode step's lengths)."""
    _cuda(k_cache, v_cache, pool_k, pool_v, block_table, cu_q, ctx_lens)
    _req(pool_k, torch.float32, "pool_k"); _req(pool_v, torch.float32, "pool_v")
    G, page, dk, dv = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    check(load().b200_kv_pool_update(_p(k_cache), _p(v_cache), _is_f32(k_cache), _p(pool_k), _p(pool_v), _p(block_table),
                                     block_table.shape[1], _p(cu_q), _p(ctx_lens), n_seqs, max_new, G, dk, dv, page, pool,
                                     pool_k.shape[2], _stream()), "kv_pool_update")


def gated_recurrence_workspace(max_tokens: int, max_seqs: int, W: int, device) -> torch.Tensor:
    """Workspace of the chunked scan for steps of up to max_tokens rows in up to max_seqs sequences."""
    rows = max_tokens // load().b200_gated_recurrence_chunk_rows() + max_seqs + 1
    return torch.empty(2 * rows * W, dtype=torch.float32, device=device)


def gated_recurrence_scan(u, gates, gate_bias, lam, proj, y_col: int, y_bias, cu_seq, ctx_lens, state_slots, S, out,
                          gate_c: float, max_len: int = 1, workspace=None):
    """Gated diagonal recurrence over every sequence's new rows (csrc/gated_recurrence.cu).  max_len: an upper bound of the
    new rows per sequence; prompt portions run in chunks side by side when a workspace is given."""
    _cuda(u, gates, gate_bias, lam, proj, y_bias, cu_seq, ctx_lens, state_slots, S, out, workspace)
    for t_, n_ in ((u, "u"), (gates, "gates"), (gate_bias, "gate_bias"), (lam, "lam"), (y_bias, "y_bias"), (S, "S")):
        _req(t_, torch.float32, n_)
    W = u.shape[1]
    if out.dtype != proj.dtype:
        raise B200Error("gated_recurrence_scan: projection and output share one element type")
    if workspace is not None and max_len > 8:
        check(load().b200_gated_recurrence_scan_chunked(_p(u), _p(gates), _p(gate_bias), _p(lam), _p(proj), _is_f32(proj),
                                                        proj.stride(0), y_col, _p(y_bias), _p(cu_seq), _p(ctx_lens),
                                                        _p(state_slots), _p(S), _p(out), out.stride(0), state_slots.shape[0], W,
                                                        gate_c, u.shape[0], int(max_len), _p(workspace), workspace.numel(),
                                                        _stream()), "gated_recurrence_scan_chunked")
        return out
    check(load().b200_gated_recurrence_scan(_p(u), _p(gates), _p(gate_bias), _p(lam), _p(proj), _is_f32(proj), proj.stride(0),
                                            y_col, _p(y_bias), _p(cu_seq), _p(ctx_lens), _p(state_slots), _p(S), _p(out),
                                            out.stride(0), state_slots.shape[0], W, gate_c, _stream()), "gated_recurrence_scan")
    return out


def gla_scan(x, q_col: int, k_col: int, v_col: int, z, inv_tau: float, cu_seq, ctx_lens, state_slots, S, o_raw, H, dk, dv,
             max_len: int = 0):
    """Linear attention with the decay sigmoid(z)^inv_tau per key channel and token (csrc/gated_linear_attn.cu)."""
    _cuda(x, z, cu_seq, ctx_lens, state_slots, S, o_raw)
    _req(x, torch.float32, "x"); _req(z, torch.float32, "z"); _req(S, torch.float32, "S"); _req(o_raw, torch.float32, "o_raw")
    check(load().b200_gla_scan_rows(_p(x), x.stride(0), q_col, k_col, v_col, _p(z), z.stride(0), inv_tau, _p(cu_seq), _p(ctx_lens),
                                    _p(state_slots), _p(S), _p(o_raw), state_slots.shape[0], H, dk, dv, int(max_len), _stream()),
          "gla_scan")


# ------------------------------------------- residual streams, latent attention, gated / routed feed-forward
GATED_ACTS = {"gelu_tanh": 1, "clamped_swish": 2, "silu": 3}


def embed_streams(ids, table, X, S: int, scale: float = 1.0):
    """X [T, S*D] fp32: every stream of row t = table[ids[t]] * scale."""
    _cuda(ids, table, X)
    _req(ids, torch.int32, "ids"); _req(table, torch.bfloat16, "table"); _req(X, torch.float32, "X")
    check(load().b200_embed_streams(_p(ids), _p(table), _p(X), ids.shape[0], S, table.shape[1], table.shape[0], scale,
                                    _stream()), "embed_streams")


def streams_step(X, S: int, y=None, hc_write=None, mult: float = 1.0, hc_read=None, norm=None, xb_out=None, rows=None):
    """X [T, S*D] fp32 residual streams.  y (fp32 / bf16 [T, D]) with hc_write ([in | out | mix] fp32): the streams
    take the branch output, X_t <- sum_s mix[s, t] X_s + mult * out[t] * y.  Then u = sum_t hc_read[t] X_t (None: the
    plain sum) and xb_out = tanh(alpha u) w + b with norm = (alpha [1] fp32, w, b).  rows: gather (no y)."""
    _cuda(X, y, hc_write, hc_read, xb_out, rows)
    _req(X, torch.float32, "X")
    D = X.shape[1] // S
    T = rows.shape[0] if rows is not None else (y.shape[0] if y is not None else X.shape[0])
    alpha, w, b = norm if norm is not None else (None, None, None)
    check(load().b200_streams_step(_p(y), 0 if y is None else _is_f32(y), 0 if y is None else y.stride(0), _p(X), _p(rows),
                                   _p(hc_write), mult, _p(hc_read), _p(alpha), _p(w), _p(b), _p(xb_out),
                                   0 if xb_out is None else _is_f32(xb_out), T, S, D, _stream()), "streams_step")


def rms_rows(x, w, out, eps: float):
    """out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w; x / out may be column slices of wider rows."""
    _cuda(x, w, out)
    if x.dtype != out.dtype or x.stride(1) != 1 or out.stride(1) != 1:
        raise B200Error("rms_rows: one element type, contiguous rows")
    check(load().b200_rms_rows(_p(x), _is_f32(x), x.stride(0), _p(w), _p(out), out.stride(0), x.shape[0], x.shape[1], eps,
                               _stream()), "rms_rows")
    return out


def latent_prep(proj, kv_col: int, q, kv_norm_w, positions, slots, cache, qa, H, dn, dr, R, rot_dims, half_layout: bool,
                freq, mag: float, eps: float):
    """Latent attention's cache write and rotations (csrc/latent.cu).  proj [T, ..] holds the latent and key part at
    kv_col; q [T, H*(dn+dr)]; cache [blocks, page, R+dr]; qa [T, H*(R+dr)] receives the rotated query parts."""
    _cuda(proj, q, kv_norm_w, positions, slots, cache, qa, freq)
    _req(freq, torch.float64, "freq")
    if not (proj.dtype == q.dtype == cache.dtype == qa.dtype):
        raise B200Error("latent_prep: projection, queries, cache and absorbed queries share one element type")
    check(load().b200_latent_prep(_p(proj), _is_f32(proj), proj.stride(0), kv_col, _p(q), q.stride(0), _p(kv_norm_w),
                                  _p(positions), _p(slots), _p(cache), _p(qa), qa.stride(0), proj.shape[0], H, dn, dr, R,
                                  rot_dims, 1 if half_layout else 0, _p(freq), mag, eps, _stream()), "latent_prep")


def latent_attn_covers(H: int, R: int, dr: int) -> bool:
    return LAYER_LIST_TC and bool(load().b200_latent_attn_covers(H, R, dr))


def latent_attn_prefill(qa, cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, sink, out, H, R, dr, scale,
                        tile_rows: int = 0):
    """Causal latent attention of prompt portions in the absorbed form: qa [T, H*(R+dr)], cache [blocks, 1, page, R+dr]
    (one row per token for all heads; its first R entries are the values), out [T, H*R].  bf16 shapes the tensor-core
    kernel covers run there, everything else (fp32, odd widths) on the generic kernel with one shared key head."""
    _cuda(qa, cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, sink, out)
    if qa.dtype == torch.bfloat16 and latent_attn_covers(H, R, dr) and qa.stride(0) % 8 == 0 and qa.data_ptr() % 16 == 0:
        check(load().b200_latent_attn_prefill(_p(qa), qa.stride(0), _p(cache), cache.shape[2], _p(block_table),
                                              block_table.shape[1], _p(cu_q), _p(ctx_lens), _p(tile_seq), _p(tile_q0),
                                              tile_seq.shape[0], tile_rows or attn_sink_prefill_tile(), _p(sink), _p(out),
                                              out.stride(0), H, R, dr, scale, _stream()), "latent_attn_prefill")
        return out
    return attn_sink_prefill(qa, -1, cache, cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, sink, out, H, 1, R + dr, R,
                             scale, tile_rows=tile_rows, v_ld=R + dr)


def latent_attn_decode_splits(B: int, H: int, max_len: int) -> int:
    return load().b200_latent_attn_decode_splits(B, H, max_len)


def latent_attn_decode_workspace(B: int, H: int, R: int, num_splits: int, device) -> Optional[torch.Tensor]:
    n = load().b200_latent_attn_decode_workspace_bytes(B, H, R, num_splits)
    return torch.empty((n + 3) // 4, dtype=torch.float32, device=device) if n else None


def latent_attn_decode(qa, cache, block_table, seq_lens, sink, out, H, R, dr, scale, num_splits: int = 1, workspace=None):
    """The same for one new row per sequence (row b sees keys [0, seq_lens[b])).  num_splits > 1 (tensor-core kernel
    only): the keys of every row are cut into that many ranges, merged by a second launch."""
    _cuda(qa, cache, block_table, seq_lens, sink, out, workspace)
    if qa.dtype == torch.bfloat16 and latent_attn_covers(H, R, dr) and qa.stride(0) % 8 == 0 and qa.data_ptr() % 16 == 0:
        if workspace is None:
            num_splits = 1
        check(load().b200_latent_attn_decode(_p(qa), qa.stride(0), _p(cache), cache.shape[2], _p(block_table),
                                             block_table.shape[1], _p(seq_lens), seq_lens.shape[0], _p(sink), _p(out),
                                             out.stride(0), H, R, dr, scale, num_splits, _p(workspace), _stream()),
              "latent_attn_decode")
        return out
    return attn_sink_decode(qa, -1, cache, cache, block_table, seq_lens, sink, out, H, 1, R + dr, R, scale, v_ld=R + dr)


def simt_group_rows() -> int:
    return load().b200_simt_group_rows()


def linear_simt_grouped(x, w, out, M, N, K, ldx, ldw, ldy, batch=1, bsx=0, bsw=0, bsy=0, row_pair=None, top_k=1,
                        tile_expert=None, num_tiles=None, n_real=0, w_expert=0, row_scale=None, act: int = 0,
                        limit: float = 0.0):
    _cuda(x, w, out, row_pair, tile_expert, num_tiles, row_scale)
    if w.dtype != torch.bfloat16:
        raise B200Error("linear_simt_grouped: bf16 weights")
    check(load().b200_linear_simt_grouped(_p(x), _is_f32(x), _p(w), _p(out), _is_f32(out), M, N, K, ldx, ldw, ldy, batch,
                                          bsx, bsw, bsy, _p(row_pair), top_k, _p(tile_expert), _p(num_tiles), n_real,
                                          w_expert, _p(row_scale), act, limit, _stream()), "linear_simt_grouped")
    return out


def head_linear(x, w, out, H: int, n: int, k: int, x_head: int, out_head: int):
    """Per-head linear: out[t, h*out_head : +n] = w[h] (n x k, contiguous) @ x[t, h*x_head : +k] for every head.
    bf16 prompt-sized steps with k a multiple of 64 and 16-byte aligned head slices: one tcgen05 GEMM per head over
    strided views; otherwise ONE batched CUDA-core launch."""
    if (x.dtype == torch.bfloat16 and x.shape[0] > TC_HEAD_LINEAR_MIN_ROWS and H <= TC_HEAD_LINEAR_MAX_HEADS
            and _tc_gemm_ok(x, w, out, k) and x_head % 8 == 0 and (n * k) % 8 == 0
            and (out_head * out.element_size()) % 16 == 0):
        if not w.is_contiguous():
            raise B200Error("head_linear: the per-head matrices must be contiguous")
        check(load().b200_gemm_bf16_heads(_p(x), _p(w), _p(out), x.shape[0], n, k, x.stride(0), out.stride(0), H, x_head,
                                          out_head, _is_f32(out), _stream()), "gemm_heads")
        return out
    return linear_simt_grouped(x, w, out, x.shape[0], n, k, x.stride(0), k, out.stride(0), batch=H, bsx=x_head, bsw=n * k,
                               bsy=out_head)


TC_HEAD_LINEAR_MAX_HEADS = 128
TC_HEAD_LINEAR_MIN_ROWS = 256      # decode-sized steps: ONE batched CUDA-core launch beats H short tensor-core launches


def _tc_gemm_ok(x, w, out, K) -> bool:
    return (LAYER_LIST_TC and x.dtype == torch.bfloat16 and K % 64 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and (out.stride(0) * out.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0)


TC_GATED_ACTS = {"gelu_tanh": 1, "clamped_swish": 2}


def gated_linear(x, w_interleaved, out, act: str, limit: float = 0.0):
    """out = act(x @ gate.T) (*) (x @ up.T) with interleaved gate / up rows (weights._interleave_rows); the
    activation is computed in fp32 from the fp32 accumulators and rounded once.  bf16 in and out with K a multiple
    of 64: the tcgen05 GEMM with the activation in its epilogue; otherwise the CUDA-core kernel."""
    M, K = x.shape
    N = w_interleaved.shape[0] // 2
    if out.dtype == torch.bfloat16 and act in TC_GATED_ACTS and _tc_gemm_ok(x, w_interleaved, out, K):
        timed = TIMER is not None and not torch.cuda.is_current_stream_capturing()
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        check(load().b200_gemm_bf16_gated(_p(x), _p(w_interleaved), _p(out), M, 2 * N, K, x.stride(0), w_interleaved.stride(0),
                                          out.stride(0), TC_GATED_ACTS[act], limit, _stream()), "gemm_gated")
        if timed:
            e1.record()
            TIMER.records.append(("gemm_prefill" if M > 256 else "gemm_decode", 4.0 * M * N * K,
                                  2.0 * (2 * N * K + M * K) + 2.0 * M * N, e0, e1))
        return out
    return linear_simt_grouped(x, w_interleaved, out, M, N, K, x.stride(0), w_interleaved.stride(0), out.stride(0),
                               act=GATED_ACTS[act], limit=limit)


def moe_route_biased(logits, correction, top_k: int, scale: float, out_ids, out_w, num_experts: int):
    _cuda(logits, correction, out_ids, out_w)
    _req(logits, torch.float32, "logits")
    check(load().b200_moe_route_biased(_p(logits), logits.stride(0), _p(correction), _p(out_ids), _p(out_w),
                                       logits.shape[0], num_experts, top_k, scale, _stream()), "moe_route_biased")


class RoutedWorkspace:
    """Device buffers of one routed feed-forward (sized for max_tokens tokens, shared by every layer): pair
    bookkeeping of moe_align with 64-row tiles, the experts' hidden rows and their weighted outputs (fp32)."""

    def __init__(self, max_tokens: int, top_k: int, e_total: int, D: int, ff: int, act_dtype, device):
        self.bx = simt_group_rows()
        n_pairs = max_tokens * top_k
        self.capacity = max(moe_capacity_rows(n_pairs, e_total, bx) for bx in (32, 64, 128, 256))
        self.xp = None            # gathered input rows of the tensor-core path, allocated at its first use
        i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=device)   # noqa: E731
        self.logits = torch.empty(max_tokens, -(-e_total // 128) * 128, dtype=torch.float32, device=device)
        self.topk_ids, self.topk_w = i32(n_pairs), torch.empty(n_pairs, dtype=torch.float32, device=device)
        self.pair_row, self.row_pair = i32(n_pairs), i32(self.capacity)
        self.row_weight = torch.empty(self.capacity, dtype=torch.float32, device=device)
        self.tile_expert, self.num_tiles = i32(self.capacity // self.bx + 1), torch.zeros(2, dtype=torch.int32, device=device)
        self.act = torch.empty(self.capacity * ff, dtype=act_dtype, device=device)
        self.yp = torch.empty(self.capacity, D, dtype=torch.float32, device=device)
        self.shared = torch.empty(max_tokens, D, dtype=torch.float32, device=device)


ROUTED_LAUNCHES = 6
TC_GROUPED_ACTS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}


def routed_experts(x, router, correction, w13, w2, ws: RoutedWorkspace, out, n_real: int, n_identity: int, top_k: int,
                   scale: float, ff: int, limit: float, shared=None, sigmoid: bool = False, renormalize: bool = True,
                   weight_on: str = "output", act: str = "clamped_swish"):
    """out[t] (fp32) = sum over the top_k chosen router outputs of weight * expert(x[t]) (identity experts return
    x[t]) + shared[t].  router [n_real + n_identity, D]; w13 [n_real * 2 ff, D] interleaved; w2 [n_real * D, ff];
    shared: the shared expert's output rows (fp32) or None.  Six launches, no host synchronisation.
    sigmoid / renormalize: how the router scores and weights are formed (moe_biased.cu); weight_on "input": the sum
    is over expert(weight * x[t]) -- the weight scales the gathered input row (tensor cores) or the accumulators before
    the activation (CUDA cores) and the output rows are not scaled; act: the experts' gate activation."""
    T, D = x.shape
    E = n_real + n_identity
    n_pairs = T * top_k
    act_name = act
    # tensor cores when both expert products fit the grouped tcgen05 GEMM (bf16, K multiples of 64, 256-row weight pairs)
    tc = (LAYER_LIST_TC and x.dtype == torch.bfloat16 and n_real > 0 and D % 256 == 0 and ff % 128 == 0 and x.is_contiguous()
          and w13.stride(0) == D and w2.stride(0) == ff)
    bx = moe_block_x(n_pairs, E) if tc else ws.bx
    cap = moe_capacity_rows(n_pairs, E, bx)
    if cap > ws.capacity:
        raise B200Error(f"routed_experts: {T} tokens exceed the workspace ({ws.capacity} rows)")
    L, st = load(), _stream()
    lg = ws.logits[:T]
    # fp32 logits; a router padded to whole weight tiles (weights.load_layer_list) takes the tensor-core GEMM in bf16
    linear(x, router, lg, force_simt=router.shape[0] % 128 != 0)
    w_in = weight_on == "input"
    if w_in and n_identity:
        raise B200Error("routed_experts: identity experts with input weights are not defined")
    check(L.b200_moe_route_scored(_p(lg), lg.stride(0), _p(correction), _p(ws.topk_ids), _p(ws.topk_w), T, E, top_k, scale,
                                  1 if sigmoid else 0, 1 if renormalize else 0, st), "moe_route_scored")
    check(L.b200_moe_align(_p(ws.topk_ids), _p(ws.topk_w), n_pairs, E, bx, cap, _p(ws.pair_row), _p(ws.row_pair),
                           _p(ws.row_weight), _p(ws.tile_expert), _p(ws.num_tiles), st), "moe_align")
    act = ws.act[:cap * ff].view(cap, ff)
    if tc:
        if ws.xp is None:
            ws.xp = torch.empty(ws.capacity, D, dtype=torch.bfloat16, device=x.device)
        check(L.b200_moe_gather_scaled(_p(x), _p(ws.row_pair), _p(ws.num_tiles), _p(ws.xp), D, top_k, cap,
                                       _p(ws.row_weight) if w_in else None, st), "moe_gather")
        check(L.b200_moe_grouped_gemm_ex(_p(ws.xp), _p(w13), _p(act), cap, 2 * ff, D, n_real, D, D, ff, None,
                                         _p(ws.tile_expert), _p(ws.num_tiles), bx, 1, TC_GROUPED_ACTS[act_name], limit, 0,
                                         st), "moe_grouped_gemm(gate_up)")
        check(L.b200_moe_grouped_gemm_ex(_p(act), _p(w2), _p(ws.yp), cap, D, ff, n_real, ff, ff, D,
                                         None if w_in else _p(ws.row_weight),
                                         _p(ws.tile_expert), _p(ws.num_tiles), bx, 0, 0, 0.0, 1, st), "moe_grouped_gemm(down)")
    elif n_real:
        check(L.b200_linear_simt_grouped_ex(_p(x), _is_f32(x), _p(w13), _p(act), _is_f32(act), cap, ff, D, x.stride(0),
                                            w13.stride(0), ff, 1, 0, 0, 0, _p(ws.row_pair), top_k, _p(ws.tile_expert),
                                            _p(ws.num_tiles), n_real, 2 * ff * w13.stride(0),
                                            _p(ws.row_weight) if w_in else None, GATED_ACTS[act_name], limit, 1 if w_in else 0,
                                            st), "linear_simt_grouped(gate_up)")
        linear_simt_grouped(act, w2, ws.yp, cap, D, ff, ff, w2.stride(0), D, tile_expert=ws.tile_expert,
                            num_tiles=ws.num_tiles, n_real=n_real, w_expert=D * w2.stride(0),
                            row_scale=None if w_in else ws.row_weight)
    check(L.b200_moe_combine_mixed(_p(ws.yp), 1, D, _p(ws.pair_row), _p(ws.topk_ids), _p(ws.topk_w), _p(x), _is_f32(x),
                                   x.stride(0), _p(shared), 0 if shared is None else shared.stride(0), _p(out), out.stride(0),
                                   T, D, top_k, n_real, st), "moe_combine_mixed")
    return out
