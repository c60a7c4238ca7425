"""Side benchmark of the layer-list family (Vodavik, Danipel, Resevik, Dotorax) beside the closest existing model of equal layer
sizes (a Llama-class decoder; for Resevik also Vodavik, the other design with attention and recurrent-state layers).

`python bench.py --family vodavik|danipel|resevik|dotorax` prints ONE JSON line (not the serving benchmark's line; that workload and its
contract are untouched).  Random weights, synthetic tokens.  Two kinds of numbers:

  model:   prefill tokens/s (prompts of `prompt` tokens, `seqs` at a time through runner.prefill) and decode tokens/s
           (`batch` rows at context `prompt`, CUDA-graph steps through runner.decode), both families, same sizes.
  kernels: every kernel of the new family in isolation next to the like kernel of the Llama path, CUDA events around
           the launch, L2 flushed before each timed launch, median of `iters`; achieved bytes/s or FLOP/s over the
           measured peaks (MEASURED_PEAKS.json) = fraction of roofline, and the ratio of the two fractions.
"""
from __future__ import annotations

import json
import statistics
import sys
import time
from pathlib import Path

import numpy as np
import torch

from . import ops
from .config import (AttentionSpec, EngineConfig, GatedLinearAttentionSpec, GatedRecurrenceSpec, LatentAttentionSpec,
                     LayerListConfig, LayerSpec, LinearAttentionSpec, MLPSpec, MLSTMSpec, ModelConfig, MoESpec, RotarySpec,
                     SideBySideSpec)

ROOT = Path(__file__).resolve().parent.parent
SIZES = {
    # name: width, heads, kv_heads, head width, ff, vocab
    "2k": (2048, 16, 4, 128, 8192, 32000),
    "4k": (4096, 32, 8, 128, 14336, 32000),
}


# Danipel at the same widths: latent 512 + 64 rotated (the cache row), heads 128 + 64 wide with 128-wide values, a
# query latent of 3/8 of the width, 8 routed experts (2 chosen, 2 identity outputs) of a quarter of the dense
# feed-forward's width each plus one shared expert of that width
DANIPEL = {
    # name: kv_rank, rot_dim, dim, vdim, q_rank, experts, top, identity, expert ff
    "2k": (512, 64, 128, 128, 768, 8, 2, 2, 2048),
    "4k": (512, 64, 128, 128, 1536, 8, 2, 2, 3584),
}


def danipel_config(size: str, layers: int = 4) -> LayerListConfig:
    D, H, G, hd, ff, V = SIZES[size]
    R, dr, dn, dv, qr, E, top, ident, ffe = DANIPEL[size]
    specs = []
    for i in range(layers):
        two = i % 2 == 0
        rot = RotarySpec(dims=dr, base=1e6, layout="half" if two else "interleaved", yarn_factor=0.0 if two else 8.0,
                         yarn_original=4096.0, yarn_fast=32.0, yarn_slow=1.0)
        mix = LatentAttentionSpec(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=R, scale=(dn + dr) ** -0.5, rot=rot,
                                  q_rank=qr if two else 0, sink=not two,
                                  type_name="latent_attention_2" if two else "latent_attention")
        if i in (0, layers - 1):
            mlp = MLPSpec("dense", ff, act="gelu_tanh")
        else:
            mlp = MLPSpec("moe", ffe, act="clamped_swish",
                          moe=MoESpec(experts=E, top=top, ff=ffe, limit=7.0, identity=ident, scale=2.5, shared_ff=ffe, shared_limit=7.0))
        specs.append(LayerSpec(mix, mlp))
    return LayerListConfig("Danipel", V, D, specs, norm_eps=1e-6, residual="streams", norm="tanh", streams=2,
                           residual_mult=0.7, embed_scale=1.0)


# Resevik at the same widths: half as many 128 x 128 linear-attention heads as attention heads (the recurrent layers of
# the Vodavik benchmark have the same), a sliding window of half the prompt, 8 routed experts (2 chosen) of a quarter of
# the dense feed-forward's width in every layer
RESEVIK = {
    # name: window, experts, top, expert ff
    "2k": (1024, 8, 2, 2048),
    "4k": (1024, 8, 2, 3584),
}


def resevik_config(size: str, layers: int = 4) -> LayerListConfig:
    D, H, G, hd, ff, V = SIZES[size]
    win, E, top, ffe = RESEVIK[size]
    Hm = H // 2
    decay = tuple(1.0 - 2.0 ** (-5 - 5 * i / max(1, Hm - 1)) for i in range(Hm))
    specs = []
    for i in range(layers):
        if i % 2 == 1:
            mix = AttentionSpec(H, G, hd, hd, hd ** -0.5, qk_norm=False, qkv_bias=False, sink=False, gate=False,
                                rot=RotarySpec(dims=hd // 2, base=5e5, layout="interleaved"), qk_unit_norm=True, window=win,
                                values_are_keys=True)
        elif i % 4 == 0:
            mix = LinearAttentionSpec(Hm, hd, hd, decay, feature=None, rot=RotarySpec(dims=hd, base=1e6, layout="half"),
                                      k_scale=hd ** -0.5, out_norm="per_head", gate_act="silu", type_name="retention")
        else:
            mix = LinearAttentionSpec(Hm, hd, hd, decay, feature="silu", out_norm="all_heads", gate_act="sigmoid",
                                      type_name="lightning")
        mlp = MLPSpec("moe", ffe, act="silu", moe=MoESpec(experts=E, top=top, ff=ffe, limit=0.0, score="sigmoid",
                                                          renormalize=False, weight_on="input", act="silu"))
        specs.append(LayerSpec(mix, mlp))
    return LayerListConfig("Resevik", V, D, specs, norm_eps=1e-5, residual="parallel", norm="rms", embed_scale=D ** 0.5)


# Dotorax at the same widths: window, pooled block, taps of the input convolution, taps of the recurrent branch
DOTORAX = {"2k": (512, 16, 3, 4), "4k": (1024, 16, 3, 4)}


def dotorax_config(size: str, layers: int = 4) -> LayerListConfig:
    """attention | side by side (window + pooled blocks, recurrence of the model's width) | attention on layer 0's
    keys and values | gated linear attention (half the heads, 64-wide keys, 128-wide values); clamped gated
    feed-forwards of the Llama model's width."""
    D, H, G, hd, ff, V = SIZES[size]
    win, pool, taps, conv = DOTORAX[size]
    specs = []
    for i in range(layers):
        if i % 4 in (0, 2):
            mix = AttentionSpec(H, G, hd, hd, hd ** -0.5, qk_norm=False, qkv_bias=False, sink=False, gate=True, gate_per_head=True,
                                rot=RotarySpec(dims=hd // 2, base=5e5, layout="half"), kv_from=0 if i % 4 == 2 else None)
        elif i % 4 == 1:
            left = AttentionSpec(H, G, hd, hd, hd ** -0.5, qk_norm=False, qkv_bias=False, sink=False, gate=False,
                                 rot=RotarySpec(dims=hd // 2, base=1e4, layout="interleaved"), qk_unit_norm=True, head_temp=True,
                                 window=win, pool=pool)
            mix = SideBySideSpec(left, GatedRecurrenceSpec(D, H, conv), 0.6, 0.9)
        else:
            mix = GatedLinearAttentionSpec(H // 2, hd // 2, hd, 16.0, decay_rank=16)
        specs.append(LayerSpec(mix, MLPSpec("dense", ff, act="clamped_swish", limit=7.0)))
    return LayerListConfig("Dotorax", V, D, specs, norm_eps=1e-5, residual="sandwich", norm="rms_zero_centred",
                           residual_mult=0.3, canon_taps=taps, learned_positions=True, max_position_embeddings=8192)


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]) * 1e9, float(d["bf16_tflops"]) * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def vodavik_config(size: str, layers: int = 4) -> LayerListConfig:
    D, H, G, hd, ff, V = SIZES[size]
    specs = []
    for i in range(layers):
        if i % 2 == 0:
            specs.append(LayerSpec(AttentionSpec(H, G, hd, hd, hd ** -0.5, q_temp_coef=0.1, q_temp_every=512,
                                                 kv_from=0 if i == 2 and layers > 2 else None), MLPSpec("dense", ff)))
        else:
            specs.append(LayerSpec(MLSTMSpec(H // 2, hd, hd, 15.0), None))
    return LayerListConfig("Vodavik", V, D, specs, norm_eps=1e-5, postln_alpha=2.0, logit_scale=1.0)


def llama_config(size: str, layers: int = 4) -> ModelConfig:
    D, H, G, hd, ff, V = SIZES[size]
    return ModelConfig(vocab_size=V, hidden_size=D, intermediate_size=ff, num_hidden_layers=layers, num_attention_heads=H,
                       num_key_value_heads=G, head_dim=hd, max_position_embeddings=8192, eos_token_id=2, bos_token_id=1)


class _Flush:
    def __init__(self):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self):
        self.buf.fill_(1)


def _time(fn, flush, iters=10, warm=3):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts)


def _model_numbers(mcfg, seqs, prompt, batch, decode_steps, log):
    from .engine import LLMEngine

    T = seqs * prompt
    blocks = (max(seqs, batch) * (prompt + decode_steps + 32)) // 16 + 64
    ecfg = EngineConfig(max_model_len=prompt + decode_steps + 32, max_num_seqs=max(seqs, batch), max_num_batched_tokens=T,
                        num_gpu_blocks=blocks, enable_prefix_caching=False, cuda_graph_sizes=[batch])
    eng = LLMEngine.from_engine_config(ecfg, mcfg=mcfg)
    run, s = eng.runner, eng.sched
    V = mcfg.vocab_size
    rng = np.random.RandomState(0)
    nb = (prompt + decode_steps + 31) // 16
    tables = [list(range(1 + i * nb, 1 + (i + 1) * nb)) for i in range(max(seqs, batch))]
    slots = list(range(max(seqs, batch))) if getattr(mcfg, "has_state", False) else None

    def prefill():
        chunks = [rng.randint(0, V, prompt).tolist() for _ in range(seqs)]
        run.prefill(chunks, [0] * seqs, tables[:seqs], [True] * seqs, state_slots=slots[:seqs] if slots else None)

    for _ in range(2):
        prefill()
    torch.cuda.synchronize()
    ts = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        chunks = [rng.randint(0, V, prompt).tolist() for _ in range(seqs)]
        torch.cuda.synchronize()
        e0.record()
        run.prefill(chunks, [0] * seqs, tables[:seqs], [True] * seqs, state_slots=slots[:seqs] if slots else None)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    pf = T / statistics.median(ts)
    # decode: `batch` rows at context `prompt` (the caches hold whatever the prefill left: timing only)
    last = rng.randint(0, V, batch).astype(np.int32)
    bt = np.zeros((batch, s.max_blocks_per_seq), dtype=np.int32)
    for i in range(batch):
        bt[i, :nb] = tables[i]
    st = np.asarray(slots[:batch], dtype=np.int32) if slots else None
    for k in range(3):
        run.decode(batch, last, np.full(batch, prompt + k, dtype=np.int32), bt, state_slots=st)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(decode_steps):
        run.decode(batch, last, np.full(batch, prompt + 3 + k, dtype=np.int32), bt, state_slots=st)
    e1.record()
    torch.cuda.synchronize()
    dec = batch * decode_steps / (e0.elapsed_time(e1) * 1e-3)
    log(f"  {type(run).__name__}: prefill {pf:,.0f} tok/s, decode {dec:,.0f} tok/s ({time.perf_counter() - t0:.1f}s)")
    out = {"prefill_tok_per_s": round(pf), "decode_tok_per_s": round(dec), "graph": bool(run.graphs),
           "launches_per_decode": run.launches_per_decode}
    del eng, run
    torch.cuda.empty_cache()
    return out


def _kernel_numbers(size, T, B, ctx, log):
    """Each new kernel beside its like kernel: (seconds, bytes or FLOPs, fraction of roofline)."""
    D, H, G, hd, ff, V = SIZES[size]
    hbm, flops_peak, how = _peaks()
    flush = _Flush()
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    rnd = lambda *s, dt=bf, sc=1.0: (torch.randn(*s, device=dev, dtype=f32) * sc).to(dt)   # noqa: E731
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)   # noqa: E731
    res = {}

    def put(name, new_s, new_work, like_name, like_s, like_work, kind):
        peak = hbm if kind == "bytes" else flops_peak
        fn, fl = new_work / new_s / peak, (like_work / like_s / peak if like_s else None)
        res[name] = {"us": round(new_s * 1e6, 1), "frac_of_" + how + "_" + kind: round(fn, 3), "like": like_name,
                     "like_us": round(like_s * 1e6, 1) if like_s else None, "like_frac": round(fl, 3) if fl else None,
                     "distance_ratio": round(fl / fn, 2) if fl else None}
        log(f"  {name:28s} {new_s * 1e6:9.1f} us  {fn:6.3f} of roofline | {like_name}: "
            + (f"{like_s * 1e6:9.1f} us {fl:6.3f}  -> {fl / fn:5.2f}x as far" if fl else "none"))

    # ---- norm after the sum vs add + RMSNorm
    y, x32, w = rnd(T, D, dt=f32), rnd(T, D, dt=f32), rnd(D)      # the branch output enters the sum in fp32
    xb = torch.empty(T, D, device=dev, dtype=bf)
    t_new = _time(lambda: ops.sum_layer_norm(y, x32, w, 2.0, 1e-5, x_out=x32, xb_out=xb), flush)
    xr, rr = rnd(T, D), rnd(T, D)
    t_like = _time(lambda: ops.fused_add_rms_norm(xr, rr, w, 1e-5, out=xr, residual_out=rr), flush)
    put("sum_layer_norm", t_new, T * D * 14.0, "fused_add_rms_norm", t_like, T * D * 8.0, "bytes")

    # ---- projection post-processing + page scatter vs rotation + page scatter
    nblk = (B * ctx + T) // 16 + 8
    W = (H + 2 * G) * hd + H * hd
    proj = rnd(T, W)
    kc, vc = rnd(nblk, G, 16, hd), rnd(nblk, G, 16, hd)
    bias, qn, kn = rnd((H + 2 * G) * hd), rnd(hd), rnd(hd)
    pos = i32(np.arange(T) % 4096)
    slots = i32(np.arange(T))
    t_new = _time(lambda: ops.attn_prep(proj, bias, qn, kn, pos, slots, kc, vc, H, G, hd, hd, 1e-5, 0.1, 512), flush)
    qkv = rnd(T, (H + 2 * G) * hd)
    cs = rnd(8192, hd)
    t_like = _time(lambda: ops.rope_kv_write(qkv, pos, cs, kc, vc, slots, H, G, hd), flush)
    work = T * (H + 2 * G) * hd * 4.0
    put("attn_prep", t_new, work, "rope_kv_write", t_like, work, "bytes")

    # ---- prefill attention: tensor-core kernel with sink + gate vs without
    S = max(1, T // 2048)
    L = T // S
    tile = ops.attn_prefill_tile(H, G)
    ts_, tq_ = ops.build_prefill_tiles([L] * S, tile, [0] * S)
    nb = (L + 15) // 16
    bt = i32(np.arange(S * nb).reshape(S, nb) + 1)
    cu, ctx0 = i32(np.arange(S + 1) * L), i32(np.zeros(S))
    sink = rnd(H, dt=f32)
    out = torch.empty(T, H * hd, device=dev, dtype=bf)
    gate_col = (H + 2 * G) * hd
    ts_d, tq_d, gate_v = i32(ts_), i32(tq_), proj[:, gate_col:]       # nothing but the launch inside the timed region
    t_new = _time(lambda: ops.paged_attn_prefill_ex(proj, W, kc, vc, bt, cu, ctx0, ts_d, tq_d, out, H, G, hd, hd ** -0.5,
                                                    sink=sink, gate=gate_v), flush)
    t_like = _time(lambda: ops.paged_attn_prefill(qkv, qkv.shape[1], kc, vc, bt, cu, ctx0, ts_d, tq_d, out, H, G, hd,
                                                  hd ** -0.5), flush)
    fl = 4.0 * S * (L * L / 2) * H * hd
    t_pf_like = t_like
    put("attn_prefill(sink,gate) tc", t_new, fl, "paged_attn_prefill tc", t_like, fl, "flops")
    # the generic kernel on widths no tensor-core tile fits (96 / 64), same token count
    dk, dv = 96, 64
    Wg = (H + G) * dk + G * dv + H * dv
    projg = rnd(T, Wg)
    kcg, vcg = rnd(nblk, G, 16, dk), rnd(nblk, G, 16, dv)
    outg = torch.empty(T, H * dv, device=dev, dtype=bf)
    tsg, tqg = ops.build_prefill_tiles([L] * S, 16, [0] * S)
    tsg, tqg = i32(tsg), i32(tqg)
    t_gen = _time(lambda: ops.attn_sink_prefill(projg, (H + G) * dk + G * dv, kcg, vcg, bt, cu, ctx0, tsg, tqg, sink, outg,
                                                H, G, dk, dv, dk ** -0.5), flush, iters=3, warm=1)
    flg = 2.0 * S * (L * L / 2) * H * (dk + dv)
    put("attn_sink_prefill generic", t_gen, flg, "paged_attn_prefill tc", t_pf_like, fl, "flops")

    # ---- decode attention
    nbd = (ctx + 16) // 16
    btd = i32(np.arange(B * nbd).reshape(B, nbd) % (nblk - 1) + 1)
    lens = i32(np.full(B, ctx))
    splits = ops.attn_decode_splits(B, G, ctx + 16)
    ws = ops.attn_decode_workspace(B, H, hd, splits, dev)
    outd = torch.empty(B, H * hd, device=dev, dtype=bf)
    pB, gB, qB = proj[:B], proj[:B, gate_col:], qkv[:B]
    t_new = _time(lambda: ops.paged_attn_decode(pB, W, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=splits,
                                                workspace=ws, sink=sink, gate=gB), flush)
    t_like = _time(lambda: ops.paged_attn_decode(qB, qkv.shape[1], kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5,
                                                 num_splits=splits, workspace=ws), flush)
    kvb = B * ctx * G * hd * 2 * 2.0
    t_dec_like = t_like
    put("attn_decode(sink,gate)", t_new, kvb, "paged_attn_decode", t_like, kvb, "bytes")
    outdg = torch.empty(B, H * dv, device=dev, dtype=bf)
    pgB = projg[:B]
    t_gen = _time(lambda: ops.attn_sink_decode(pgB, (H + G) * dk + G * dv, kcg, vcg, btd, lens, sink, outdg, H, G, dk, dv,
                                               dk ** -0.5), flush)
    put("attn_sink_decode generic", t_gen, B * ctx * G * (dk + dv) * 2.0, "paged_attn_decode", t_dec_like, kvb, "bytes")

    # ---- matrix-memory recurrence: prompt portions and single rows
    Hm = H // 2
    pm = rnd(T, 4 * Hm * hd, sc=0.5)
    gates = rnd(T, 2 * Hm, dt=f32)
    gb = rnd(2 * Hm)
    Z = ops.mlstm_state_slices(hd)
    nslot = max(S, B)
    Sst = torch.zeros(nslot, Hm, hd, hd, device=dev)      # [slots, H, dv, dk]
    nst, mst = torch.zeros(nslot, Hm, Z, hd, device=dev), torch.zeros(nslot, Hm, Z, device=dev)
    o_raw = torch.empty(T, Hm * hd, device=dev)
    slot_s, slot_b = i32(np.arange(S)), i32(np.arange(B))
    t_scan = _time(lambda: ops.mlstm_scan(pm, 0, Hm * hd, 2 * Hm * hd, gates, gb, cu, ctx0, slot_s, Sst, nst, mst, o_raw,
                                          Hm, hd, hd, 15.0, max_len=L), flush, iters=3, warm=1)
    put("mlstm_scan prefill", t_scan, 6.0 * T * Hm * hd * hd, "paged_attn_prefill tc", t_pf_like, fl, "flops")
    cud, ctxd = i32(np.arange(B + 1)), i32(np.full(B, ctx))
    pmB, gatesB, orB = pm[:B], gates[:B], o_raw[:B]
    t_step = _time(lambda: ops.mlstm_scan(pmB, 0, Hm * hd, 2 * Hm * hd, gatesB, gb, cud, ctxd, slot_b, Sst, nst, mst,
                                          orB, Hm, hd, hd, 15.0), flush)
    put("mlstm_scan decode", t_step, B * Hm * hd * hd * 8.0, "paged_attn_decode", t_dec_like, kvb, "bytes")
    mo = torch.empty(T, Hm * hd, device=dev, dtype=bf)
    nw = rnd(Hm * hd)
    t_new = _time(lambda: ops.mlstm_out(o_raw, pm, 3 * Hm * hd, nw, mo, Hm, hd, 1e-5), flush)
    act2 = rnd(T, 2 * Hm * hd)
    t_like2 = _time(lambda: ops.silu_and_mul(act2, out=mo), flush)
    put("mlstm_out", t_new, T * Hm * hd * 8.0, "silu_and_mul", t_like2, T * Hm * hd * 6.0, "bytes")

    # ---- feed-forward up projection with its activation in the epilogue
    xin, wu = rnd(T, D), rnd(ff, D, sc=0.02)
    au = torch.empty(T, ff, device=dev, dtype=bf)
    t_new = _time(lambda: ops.linear(xin, wu, au, relu2=True), flush)
    wgu = rnd(2 * ff, D, sc=0.02)
    t_like3 = _time(lambda: ops.gemm_silu_mul(xin, wgu, out=au), flush)
    put("gemm + relu^2", t_new, 2.0 * T * ff * D, "gemm + SiLU*mul", t_like3, 4.0 * T * ff * D, "flops")
    return res


def _kernel_numbers_danipel(size, T, B, ctx, log):
    """Danipel's kernels beside the like kernels of the Llama-class path (dense and routed) at equal sizes."""
    from .weights import _interleave_rows

    D, H, G, hd, ff, V = SIZES[size]
    R, dr, dn, dv, qr, E, top, ident, ffe = DANIPEL[size]
    W = R + dr
    hbm, flops_peak, how = _peaks()
    flush = _Flush()
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    rnd = lambda *s, dt=bf, sc=1.0: (torch.randn(*s, device=dev, dtype=f32) * sc).to(dt)   # noqa: E731
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)   # noqa: E731
    res = {}

    def put(name, new_s, new_work, like_name, like_s, like_work, kind):
        peak = hbm if kind == "bytes" else flops_peak
        fn, fl = new_work / new_s / peak, like_work / like_s / peak
        res[name] = {"us": round(new_s * 1e6, 1), "frac_of_" + how + "_" + kind: round(fn, 3), "like": like_name,
                     "like_us": round(like_s * 1e6, 1), "like_frac": round(fl, 3), "distance_ratio": round(fl / fn, 2)}
        log(f"  {name:34s} {new_s * 1e6:9.1f} us  {fn:6.3f} of roofline | {like_name}: {like_s * 1e6:9.1f} us {fl:6.3f}"
            f"  -> {fl / fn:5.2f}x as far")

    # ---- two residual streams: write-back + read + tanh norm in one pass, vs add + RMSNorm
    S2 = 2
    X = rnd(T, S2 * D, dt=f32)
    y = rnd(T, D, dt=f32)
    hc = rnd(2 * S2 + S2 * S2, dt=f32)
    alpha, w, b = torch.full((1,), 0.5, device=dev), rnd(D), rnd(D)
    xb = torch.empty(T, D, device=dev, dtype=bf)
    t_new = _time(lambda: ops.streams_step(X, S2, y=y, hc_write=hc, mult=0.7, hc_read=hc, norm=(alpha, w, b), xb_out=xb), flush)
    xr, rr = rnd(T, D), rnd(T, D)
    t_like = _time(lambda: ops.fused_add_rms_norm(xr, rr, w, 1e-5, out=xr, residual_out=rr), flush)
    put("streams_step (2 streams)", t_new, T * D * (S2 * 8.0 + 4 + 2), "fused_add_rms_norm", t_like, T * D * 8.0, "bytes")

    # ---- latent norm + rotations + cache row vs rotation + page scatter
    nblk = (B * ctx + T) // 16 + 8
    proj = rnd(T, H * (dn + dr) + W)
    cache = rnd(nblk, 1, 16, W)
    qa = torch.empty(T, H * W, device=dev, dtype=bf)
    pos, slots = i32(np.arange(T) % 4096), i32(np.arange(T))
    freq = torch.tensor(RotarySpec(dims=dr, base=1e6).frequencies()[0], dtype=torch.float64, device=dev)
    kvw = rnd(R)
    t_new = _time(lambda: ops.latent_prep(proj, H * (dn + dr), proj[:, :H * (dn + dr)], kvw, pos, slots, cache, qa, H, dn, dr, R, dr,
                                          False, freq, 1.0, 1e-6), flush)
    qkv = rnd(T, (H + 2 * G) * hd)
    kc, vc = rnd(nblk, G, 16, hd), rnd(nblk, G, 16, hd)
    cs = rnd(8192, hd)
    t_like = _time(lambda: ops.rope_kv_write(qkv, pos, cs, kc, vc, slots, H, G, hd), flush)
    put("latent_prep", t_new, T * (W + H * dr) * 4.0, "rope_kv_write", t_like, T * (H + 2 * G) * hd * 4.0, "bytes")

    # ---- per-head absorption of W_uk into the queries / W_uv after the attention vs one plain GEMM
    ukt = rnd(H, R, dn, sc=0.05)
    t_new = _time(lambda: ops.head_linear(proj, ukt, qa, H, n=R, k=dn, x_head=dn + dr, out_head=W), flush)
    wq = rnd((H + 2 * G) * hd, D, sc=0.02)
    xin = rnd(T, D)
    t_like = _time(lambda: ops.gemm(xin, wq, out=qkv), flush)
    put("query absorption (H GEMMs)", t_new, 2.0 * T * H * dn * R, "qkv GEMM", t_like, 2.0 * T * (H + 2 * G) * hd * D, "flops")
    o_lat = rnd(T, H * R)
    uv = rnd(H * dv, R, sc=0.05)
    mo = torch.empty(T, H * dv, device=dev, dtype=bf)
    t_new = _time(lambda: ops.head_linear(o_lat, uv, mo, H, n=dv, k=R, x_head=R, out_head=dv), flush)
    put("value expansion (H GEMMs)", t_new, 2.0 * T * H * dv * R, "qkv GEMM", t_like, 2.0 * T * (H + 2 * G) * hd * D, "flops")

    # ---- attention over the latent cache vs the Llama-class kernels
    Sq = max(1, T // 2048)
    L = T // Sq
    nb = (L + 15) // 16
    bt = i32(np.arange(Sq * nb).reshape(Sq, nb) + 1)
    cu, ctx0 = i32(np.arange(Sq + 1) * L), i32(np.zeros(Sq))
    ts_, tq_ = ops.build_prefill_tiles([L] * Sq, ops.attn_sink_prefill_tile(), [0] * Sq)
    ts_d, tq_d = i32(ts_), i32(tq_)
    sink = rnd(H, dt=f32)
    t_new = _time(lambda: ops.latent_attn_prefill(qa, cache, bt, cu, ctx0, ts_d, tq_d, sink, o_lat, H, R, dr, W ** -0.5), flush,
                  iters=5, warm=2)
    tile = ops.attn_prefill_tile(H, G)
    tl, tql = ops.build_prefill_tiles([L] * Sq, tile, [0] * Sq)
    tl, tql = i32(tl), i32(tql)
    out = torch.empty(T, H * hd, device=dev, dtype=bf)
    t_like = _time(lambda: ops.paged_attn_prefill(qkv, qkv.shape[1], kc, vc, bt, cu, ctx0, tl, tql, out, H, G, hd, hd ** -0.5), flush)
    pairs = Sq * (L * L / 2)
    put("latent attention prefill", t_new, 2.0 * pairs * H * (W + R), "paged_attn_prefill tc", t_like, 4.0 * pairs * H * hd, "flops")
    nbd = (ctx + 16) // 16
    btd = i32(np.arange(B * nbd).reshape(B, nbd) % (nblk - 1) + 1)
    lens = i32(np.full(B, ctx))
    qaB, olB = qa[:B], o_lat[:B]
    lsp = ops.latent_attn_decode_splits(B, H, ctx + 16)
    lws = ops.latent_attn_decode_workspace(B, H, R, 16, dev)
    t_new = _time(lambda: ops.latent_attn_decode(qaB, cache, btd, lens, sink, olB, H, R, dr, W ** -0.5, num_splits=lsp,
                                                 workspace=lws), flush)
    splits = ops.attn_decode_splits(B, G, ctx + 16)
    ws = ops.attn_decode_workspace(B, H, hd, splits, dev)
    outd = torch.empty(B, H * hd, device=dev, dtype=bf)
    qB = qkv[:B]
    t_like = _time(lambda: ops.paged_attn_decode(qB, qkv.shape[1], kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5,
                                                 num_splits=splits, workspace=ws), flush)
    put("latent attention decode", t_new, B * ctx * W * 2.0, "paged_attn_decode", t_like, B * ctx * G * hd * 4.0, "bytes")
    res["latent attention decode"]["tflops"] = round(2.0 * B * ctx * H * (W + R) / t_new / 1e12, 1)

    # ---- gated feed-forward: activation in the GEMM's epilogue
    wgu = rnd(2 * ff, D, sc=0.02)
    au = torch.empty(T, ff, device=dev, dtype=bf)
    t_new = _time(lambda: ops.gated_linear(xin, wgu, au, "gelu_tanh"), flush)
    t_like = _time(lambda: ops.gemm_silu_mul(xin, wgu, out=au), flush)
    put("gate_up GEMM + GELU*mul", t_new, 4.0 * T * ff * D, "gate_up GEMM + SiLU*mul", t_like, 4.0 * T * ff * D, "flops")

    # ---- routed experts (router, choice, pair grouping, grouped GEMMs, combine) vs the Mixtral path at equal sizes
    for rows, tag in ((T, "prefill"), (B, "decode")):
        rws = ops.RoutedWorkspace(rows, top, E + ident, D, ffe, bf, dev)
        router, corr = torch.zeros(128, D, device=dev, dtype=bf), rnd(E + ident, dt=f32, sc=0.01)
        router[:E + ident] = rnd(E + ident, D, sc=0.05)          # zero rows up to a weight tile, as the loader stores it
        w13 = rnd(E * 2 * ffe, D, sc=0.02)
        w2 = rnd(E * D, ffe, sc=0.02)
        xr_ = xin[:rows]
        yo = torch.empty(rows, D, device=dev, dtype=f32)
        t_new = _time(lambda: ops.routed_experts(xr_, router, corr, w13, w2, rws, yo, E, ident, top, 2.5, ffe, 7.0), flush,
                      iters=5, warm=2)
        mws = ops.MoEWorkspace(rows, top, E, D, ffe, dev)
        rl = rnd(rows, ops.ROUTER_PAD)
        rw_ = ops.pad_router(router[:E].contiguous())
        yb = torch.empty(rows, D, device=dev, dtype=bf)

        def like():
            ops.gemm(xr_, rw_, out=rl)
            ops.moe_experts(xr_, rl, w13, w2, top, mws, out=yb)

        t_like = _time(like, flush, iters=5, warm=2)
        # identity outputs take a share of the pairs: count the expert products of an even spread
        share = E / (E + ident)
        put(f"routed experts ({tag})", t_new, 6.0 * rows * top * share * D * ffe, f"Mixtral experts ({tag})", t_like,
            6.0 * rows * top * D * ffe, "flops")
        del rws, mws
    return res


def _kernel_numbers_resevik(size, T, B, ctx, log):
    """Resevik's kernels beside the like kernels of the closest models (Vodavik's norm, preparation, attention and
    recurrence kernels; the Mixtral experts) at equal sizes."""
    D, H, G, hd, ff, V = SIZES[size]
    win, E, top, ffe = RESEVIK[size]
    Hm = H // 2
    hbm, flops_peak, how = _peaks()
    flush = _Flush()
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    rnd = lambda *s, dt=bf, sc=1.0: (torch.randn(*s, device=dev, dtype=f32) * sc).to(dt)   # noqa: E731
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)   # noqa: E731
    res = {}

    def put(name, new_s, new_work, like_name, like_s, like_work, kind):
        peak = hbm if kind == "bytes" else flops_peak
        fn, fl = new_work / new_s / peak, like_work / like_s / peak
        res[name] = {"us": round(new_s * 1e6, 1), "frac_of_" + how + "_" + kind: round(fn, 3), "like": like_name,
                     "like_us": round(like_s * 1e6, 1), "like_frac": round(fl, 3), "distance_ratio": round(fl / fn, 2)}
        log(f"  {name:34s} {new_s * 1e6:9.1f} us  {fn:6.3f} of roofline | {like_name}: {like_s * 1e6:9.1f} us {fl:6.3f}"
            f"  -> {fl / fn:5.2f}x as far")

    # ---- residual sum of two branch outputs + RMS norm, vs the norm after the sum of the post-norm design
    x32, ya, yb, w = rnd(T, D, dt=f32), rnd(T, D, dt=f32), rnd(T, D, dt=f32), rnd(D)
    xb = torch.empty(T, D, device=dev, dtype=bf)
    t_new = _time(lambda: ops.add_rms_norm(x32, w, 1e-5, a=ya, b=yb, x_out=x32, xb_out=xb), flush)
    t_like = _time(lambda: ops.sum_layer_norm(ya, x32, w, 2.0, 1e-5, x_out=x32, xb_out=xb), flush)
    put("add_rms_norm (2 branches)", t_new, T * D * 18.0, "sum_layer_norm", t_like, T * D * 14.0, "bytes")

    # ---- rotation + unit norm + page scatter (values = keys), vs bias + head norms + temperature + page scatter
    nblk = (B * ctx + T) // 16 + 8
    proj = rnd(T, (H + G) * hd)
    kc, vc = rnd(nblk, G, 16, hd), rnd(nblk, G, 16, hd)
    pos, slots = i32(np.arange(T) % 4096), i32(np.arange(T))
    freq = torch.tensor(RotarySpec(dims=hd // 2, base=5e5).frequencies()[0], dtype=torch.float64, device=dev)
    t_new = _time(lambda: ops.rot_prep(proj, 0, H * hd, -1, pos, slots, proj, kc, vc, H, G, hd, hd, paged=True,
                                       rot_dims=hd // 2, half_layout=False, freq=freq, unit_norm=True, eps=1e-5), flush)
    Wv = (H + 2 * G) * hd + H * hd
    projv = rnd(T, Wv)
    bias, qn, kn = rnd((H + 2 * G) * hd), rnd(hd), rnd(hd)
    t_prep = _time(lambda: ops.attn_prep(projv, bias, qn, kn, pos, slots, kc, vc, H, G, hd, hd, 1e-5, 0.1, 512), flush)
    put("rot_prep (attention)", t_new, T * (2 * H + 3 * G) * hd * 2.0, "attn_prep", t_prep, T * (H + 2 * G) * hd * 4.0, "bytes")
    # the recurrent mixers' preparation: bf16 rows in, fp32 q | k | v rows out
    pl = rnd(T, 4 * Hm * hd, sc=0.5)
    x32l = torch.empty(T, 3 * Hm * hd, device=dev)
    freql = torch.tensor(RotarySpec(dims=hd, base=1e6).frequencies()[0], dtype=torch.float64, device=dev)
    kcl, vcl = Hm * hd, 2 * Hm * hd
    t_new = _time(lambda: ops.rot_prep(pl, 0, kcl, vcl, pos, None, x32l, x32l[:, kcl:], x32l[:, vcl:], Hm, Hm, hd, hd, paged=False,
                                       rot_dims=hd, half_layout=True, freq=freql, k_mul=hd ** -0.5), flush)
    put("rot_prep (retention, fp32 out)", t_new, T * 3 * Hm * hd * 6.0, "attn_prep", t_prep, T * (H + 2 * G) * hd * 4.0, "bytes")

    # ---- prefill attention in a window: the tcgen05 kernel with and without the window
    S = max(1, T // 2048)
    L = T // S
    tile = ops.attn_prefill_tile(H, G)
    ts_, tq_ = ops.build_prefill_tiles([L] * S, tile, [0] * S)
    nb = (L + 15) // 16
    bt = i32(np.arange(S * nb).reshape(S, nb) + 1)
    cu, ctx0 = i32(np.arange(S + 1) * L), i32(np.zeros(S))
    out = torch.empty(T, H * hd, device=dev, dtype=bf)
    ts_d, tq_d = i32(ts_), i32(tq_)
    Wp = proj.shape[1]
    t_new = _time(lambda: ops.paged_attn_prefill_ex(proj, Wp, kc, vc, bt, cu, ctx0, ts_d, tq_d, out, H, G, hd, hd ** -0.5,
                                                    window=win), flush)
    sink = rnd(H, dt=f32)
    gate_col = (H + 2 * G) * hd
    gate_v = projv[:, gate_col:]
    t_like = _time(lambda: ops.paged_attn_prefill_ex(projv, Wv, kc, vc, bt, cu, ctx0, ts_d, tq_d, out, H, G, hd, hd ** -0.5,
                                                     sink=sink, gate=gate_v), flush)
    pairs_w = S * sum(min(i + 1, win) for i in range(L))
    put("attention prefill, window tc", t_new, 4.0 * pairs_w * H * hd, "attention prefill, sink + gate tc", t_like,
        4.0 * S * (L * L / 2) * H * hd, "flops")

    # ---- decode attention in a window
    nbd = (ctx + 16) // 16
    btd = i32(np.arange(B * nbd).reshape(B, nbd) % (nblk - 1) + 1)
    lens = i32(np.full(B, ctx))
    outd = torch.empty(B, H * hd, device=dev, dtype=bf)
    sp_w = ops.attn_decode_splits(B, G, min(ctx + 16, win))
    ws_w = ops.attn_decode_workspace(B, H, hd, sp_w, dev)
    pB = proj[:B]
    t_new = _time(lambda: ops.paged_attn_decode(pB, Wp, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=sp_w,
                                                workspace=ws_w, window=win), flush)
    splits = ops.attn_decode_splits(B, G, ctx + 16)
    ws = ops.attn_decode_workspace(B, H, hd, splits, dev)
    pvB, gB = projv[:B], projv[:B, gate_col:]
    t_like = _time(lambda: ops.paged_attn_decode(pvB, Wv, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=splits,
                                                 workspace=ws, sink=sink, gate=gB), flush)
    put("attention decode, window", t_new, B * min(ctx, win) * G * hd * 4.0, "attention decode, sink + gate", t_like,
        B * ctx * G * hd * 4.0, "bytes")

    # ---- decayed linear attention vs the matrix-memory recurrence: prompt portions and single rows
    x32l.normal_(0.0, 0.3)
    decay = torch.tensor([1.0 - 2.0 ** (-5 - 5 * i / max(1, Hm - 1)) for i in range(Hm)], device=dev)
    nslot = max(S, B)
    Sst = torch.zeros(nslot, Hm, hd, hd, device=dev)
    o_raw = torch.empty(T, Hm * hd, device=dev)
    slot_s, slot_b = i32(np.arange(S)), i32(np.arange(B))
    t_new = _time(lambda: ops.linattn_scan(x32l, 0, kcl, vcl, decay, cu, ctx0, slot_s, Sst, o_raw, Hm, hd, hd, max_len=L), flush,
                  iters=3, warm=1)
    pm = rnd(T, 4 * Hm * hd, sc=0.5)
    gates, gb = rnd(T, 2 * Hm, dt=f32), rnd(2 * Hm)
    Z = ops.mlstm_state_slices(hd)
    nst, mst = torch.zeros(nslot, Hm, Z, hd, device=dev), torch.zeros(nslot, Hm, Z, device=dev)
    Sm = torch.zeros(nslot, Hm, hd, hd, device=dev)
    t_like = _time(lambda: ops.mlstm_scan(pm, 0, Hm * hd, 2 * Hm * hd, gates, gb, cu, ctx0, slot_s, Sm, nst, mst, o_raw, Hm, hd, hd,
                                          15.0, max_len=L), flush, iters=3, warm=1)
    fma_peak = 148 * 128 * 2 * 1.9e9          # fp32 FMA rate: the recurrence's products are fp32 by the exactness rule
    wl = 6.0 * T * Hm * hd * hd
    res["linattn_scan prefill (chunk)"] = {"us": round(t_new * 1e6, 1), "frac_of_fp32_fma": round(wl / t_new / fma_peak, 3),
                                           "like": "mlstm_scan prefill (chunk)", "like_us": round(t_like * 1e6, 1),
                                           "like_frac": round(wl / t_like / fma_peak, 3), "distance_ratio": round(t_new / t_like, 2)}
    log(f"  linattn_scan prefill (chunk)       {t_new * 1e6:9.1f} us  {wl / t_new / fma_peak:6.3f} of fp32 FMA | mlstm_scan: "
        f"{t_like * 1e6:9.1f} us {wl / t_like / fma_peak:6.3f}  -> {t_new / t_like:5.2f}x as far")
    cud, ctxd = i32(np.arange(B + 1)), i32(np.full(B, ctx))
    xB, orB, pmB, gatesB = x32l[:B], o_raw[:B], pm[:B], gates[:B]
    t_new = _time(lambda: ops.linattn_scan(xB, 0, kcl, vcl, decay, cud, ctxd, slot_b, Sst, orB, Hm, hd, hd), flush)
    t_like = _time(lambda: ops.mlstm_scan(pmB, 0, Hm * hd, 2 * Hm * hd, gatesB, gb, cud, ctxd, slot_b, Sm, nst, mst, orB, Hm, hd, hd,
                                          15.0), flush)
    put("linattn_scan decode", t_new, B * Hm * hd * hd * 8.0, "mlstm_scan decode", t_like, B * Hm * hd * hd * 8.0, "bytes")
    mo = torch.empty(T, Hm * hd, device=dev, dtype=bf)
    nw = rnd(Hm * hd)
    t_new = _time(lambda: ops.linattn_out(o_raw, pl, 3 * Hm * hd, nw, mo, Hm, hd, 1e-5, True, "sigmoid"), flush)
    t_like = _time(lambda: ops.mlstm_out(o_raw, pm, 3 * Hm * hd, nw, mo, Hm, hd, 1e-5), flush)
    put("linattn_out (all heads)", t_new, T * Hm * hd * 8.0, "mlstm_out", t_like, T * Hm * hd * 8.0, "bytes")
    t_new = _time(lambda: ops.linattn_out(o_raw, pl, 3 * Hm * hd, None, mo, Hm, hd, 1e-5, False, "silu"), flush)
    put("linattn_out (per head)", t_new, T * Hm * hd * 8.0, "mlstm_out", t_like, T * Hm * hd * 8.0, "bytes")

    # ---- sigmoid-routed experts weighted on their input vs the Mixtral path at equal sizes
    xin = rnd(T, D)
    for rows, tag in ((T, "prefill"), (B, "decode")):
        rws = ops.RoutedWorkspace(rows, top, E, D, ffe, bf, dev)
        router = torch.zeros(128, D, device=dev, dtype=bf)
        router[:E] = rnd(E, D, sc=0.05)
        w13 = rnd(E * 2 * ffe, D, sc=0.02)
        w2 = rnd(E * D, ffe, sc=0.02)
        xr_ = xin[:rows]
        yo = torch.empty(rows, D, device=dev, dtype=f32)
        t_new = _time(lambda: ops.routed_experts(xr_, router, None, w13, w2, rws, yo, E, 0, top, 1.0, ffe, 0.0, sigmoid=True,
                                                 renormalize=False, weight_on="input", act="silu"), flush, iters=5, warm=2)
        mws = ops.MoEWorkspace(rows, top, E, D, ffe, dev)
        rl = rnd(rows, ops.ROUTER_PAD)
        rw_ = ops.pad_router(router[:E].contiguous())
        ybf = torch.empty(rows, D, device=dev, dtype=bf)

        def like():
            ops.gemm(xr_, rw_, out=rl)
            ops.moe_experts(xr_, rl, w13, w2, top, mws, out=ybf)

        t_like = _time(like, flush, iters=5, warm=2)
        put(f"routed experts ({tag})", t_new, 6.0 * rows * top * D * ffe, f"Mixtral experts ({tag})", t_like,
            6.0 * rows * top * D * ffe, "flops")
        del rws, mws
    return res


def _kernel_numbers_dotorax(size, T, B, ctx, log):
    """Dotorax's kernels beside the like kernels of the closest model (Resevik: fp32 residual with a norm per layer,
    rotary window attention, decayed linear attention) at equal sizes."""
    D, H, G, hd, ff, V = SIZES[size]
    win, pool, taps, conv = DOTORAX[size]
    Hm, dkg = H // 2, hd // 2
    hbm, flops_peak, how = _peaks()
    flush = _Flush()
    dev = "cuda"
    bf, f32 = torch.bfloat16, torch.float32
    rnd = lambda *s, dt=bf, sc=1.0: (torch.randn(*s, device=dev, dtype=f32) * sc).to(dt)   # noqa: E731
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)   # noqa: E731
    res = {}

    def put(name, new_s, new_work, like_name, like_s, like_work, kind):
        peak = hbm if kind == "bytes" else flops_peak
        fn, fl = new_work / new_s / peak, like_work / like_s / peak
        res[name] = {"us": round(new_s * 1e6, 1), "frac_of_" + how + "_" + kind: round(fn, 4), "like": like_name,
                     "like_us": round(like_s * 1e6, 1), "like_frac": round(fl, 4), "distance_ratio": round(fl / fn, 2)}
        log(f"  {name:36s} {new_s * 1e6:9.1f} us  {fn:7.4f} of roofline | {like_name}: {like_s * 1e6:9.1f} us {fl:7.4f}"
            f"  -> {fl / fn:5.2f}x as far")

    S = max(1, T // 2048)
    L = T // S
    cu, ctx0, slot_s = i32(np.arange(S + 1) * L), i32(np.zeros(S)), i32(np.arange(S))
    cud, ctxd, slot_b = i32(np.arange(B + 1)), i32(np.full(B, ctx)), i32(np.arange(B))
    # ---- join (norm of the output, sum, norm of the sum) vs sum + norm of the one-norm-per-layer design
    x32, ya, yb, w, w2 = rnd(T, D, dt=f32), rnd(T, D, dt=f32), rnd(T, D, dt=f32), rnd(D, sc=0.2), rnd(D, sc=0.2)
    xb, h32 = torch.empty(T, D, device=dev, dtype=bf), torch.empty(T, D, device=dev)
    t_new = _time(lambda: ops.sandwich_join(x32, 1e-5, y=ya, post_w=w, mult=0.3, pre_w=w2, x_out=x32, h_out=h32), flush)
    t_like = _time(lambda: ops.add_rms_norm(x32, w, 1e-5, a=ya, x_out=x32, xb_out=xb), flush)
    put("sandwich_join", t_new, T * D * 16.0, "add_rms_norm (1 branch)", t_like, T * D * 14.0, "bytes")
    t_new = _time(lambda: ops.sandwich_join(x32, 1e-5, y=ya, y2=yb, ya=0.6, yb=0.9, post_w=w, mult=0.3, pre_w=w2, x_out=x32,
                                            h_out=h32), flush)
    t_like2 = _time(lambda: ops.add_rms_norm(x32, w, 1e-5, a=ya, b=yb, x_out=x32, xb_out=xb), flush)
    put("sandwich_join (2 outputs)", t_new, T * D * 20.0, "add_rms_norm (2 branches)", t_like2, T * D * 18.0, "bytes")
    # ---- input convolution with rings (+ commit) vs the same streaming norm kernel
    cw = rnd(D, taps, dt=f32, sc=0.4)
    ring = torch.zeros(max(S, B), taps - 1, D, device=dev)

    def conv_():
        ops.causal_conv(h32, cw, ring, cu, ctx0, slot_s, xb, add_input=True)
        ops.conv_commit(h32, ring, cu, ctx0, slot_s, taps)

    t_new = _time(conv_, flush)
    put("causal_conv + commit (prefill)", t_new, T * D * 6.0, "add_rms_norm (1 branch)", t_like, T * D * 14.0, "bytes")

    # ---- attention with one gate per head (half rotation): generic kernel vs the tcgen05 kernel with sink + element gate
    nblk = (B * ctx + T) // 16 + 8
    Wp = (H + 2 * G) * hd + 8
    proj = rnd(T, Wp)
    kc, vc = rnd(nblk, G, 16, hd), rnd(nblk, G, 16, hd)
    pos, slots = i32(np.arange(T) % L), i32(np.arange(T) + 16)
    freq = torch.tensor(RotarySpec(dims=hd // 2, base=5e5).frequencies()[0], dtype=torch.float64, device=dev)
    t_new = _time(lambda: ops.rot_prep(proj, 0, H * hd, (H + G) * hd, pos, slots, proj, kc, vc, H, G, hd, hd, paged=True,
                                       rot_dims=hd // 2, half_layout=True, freq=freq), flush)
    projr = rnd(T, (H + G) * hd)
    t_like = _time(lambda: ops.rot_prep(projr, 0, H * hd, -1, pos, slots, projr, kc, vc, H, G, hd, hd, paged=True,
                                        rot_dims=hd // 2, half_layout=False, freq=freq, unit_norm=True, eps=1e-5), flush)
    put("rot_prep (half, own values)", t_new, T * (2 * H + 4 * G) * hd * 2.0, "rot_prep (Resevik attention)", t_like,
        T * (2 * H + 3 * G) * hd * 2.0, "bytes")
    tile = ops.attn_sink_prefill_tile()
    ts_, tq_ = ops.build_prefill_tiles([L] * S, tile, [0] * S)
    nb = (L + 15) // 16
    bt = i32(np.arange(S * nb).reshape(S, nb) + 1)
    out = torch.empty(T, H * hd, device=dev, dtype=bf)
    ts_d, tq_d = i32(ts_), i32(tq_)
    gate_col = (H + 2 * G) * hd
    tile_tc = ops.attn_prefill_tile(H, G)
    tt_, tqq_ = ops.build_prefill_tiles([L] * S, tile_tc, [0] * S)
    tt_d, tqq_d = i32(tt_), i32(tqq_)
    t_new = _time(lambda: ops.paged_attn_prefill_ex(proj, Wp, kc, vc, bt, cu, ctx0, tt_d, tqq_d, out, H, G, hd, hd ** -0.5,
                                                    gate=proj[:, gate_col:], gate_per_head=True), flush)
    Wv = (H + 2 * G) * hd + H * hd
    projv = rnd(T, Wv)
    sink = rnd(H, dt=f32)
    t_tc = _time(lambda: ops.paged_attn_prefill_ex(projv, Wv, kc, vc, bt, cu, ctx0, tt_d, tqq_d, out, H, G, hd, hd ** -0.5,
                                                   sink=sink, gate=projv[:, gate_col:]), flush)
    full = 4.0 * S * (L * L / 2) * H * hd
    put("attention prefill, head gate", t_new, full, "attention prefill, sink + gate tc", t_tc, full, "flops")
    # ---- window + pooled blocks vs the tcgen05 kernel with a window
    per_page = -(-16 // pool)
    pk, pv = torch.zeros(nblk, G, per_page, hd, device=dev), torch.zeros(nblk, G, per_page, hd, device=dev)
    temp = rnd(H, dt=f32, sc=0.1) + 1.0
    t_pool = _time(lambda: ops.kv_pool_update(kc, vc, pk, pv, bt, cu, ctx0, S, L, pool), flush)
    lse = torch.empty(T, H, device=dev)

    def window_then_pooled():
        ops.paged_attn_prefill_ex(proj, Wp, kc, vc, bt, cu, ctx0, tt_d, tqq_d, out, H, G, hd, hd ** -0.5, window=win, lse_out=lse)
        ops.attn_sink_prefill_more(proj, kc, bt, cu, ctx0, tt_d, tqq_d, out, lse, H, G, hd, hd, hd ** -0.5, tile_tc, win, None,
                                   (pk, pv, pool))

    t_new = _time(window_then_pooled, flush)
    t_gen = _time(lambda: ops.attn_sink_prefill(proj, -1, kc, vc, bt, cu, ctx0, ts_d, tq_d, None, out, H, G, hd, hd, hd ** -0.5,
                                                window=win, head_scale=temp, pool=(pk, pv, pool)), flush, iters=3, warm=1)
    t_win = _time(lambda: ops.paged_attn_prefill_ex(projr, projr.shape[1], kc, kc, bt, cu, ctx0, tt_d, tqq_d, out, H, G, hd,
                                                    hd ** -0.5, window=win), flush)
    pairs_w = S * sum(min(i + 1, win) for i in range(L))
    pairs_p = pairs_w + S * sum(max(0, (i - win + 1) // pool) for i in range(L))
    put("attention prefill, window + pooled", t_new, 4.0 * pairs_p * H * hd, "attention prefill, window tc", t_win,
        4.0 * pairs_w * H * hd, "flops")
    put("attention prefill, window + pooled (generic kernel alone)", t_gen, 4.0 * pairs_p * H * hd, "attention prefill, window tc",
        t_win, 4.0 * pairs_w * H * hd, "flops")
    put("kv_pool_update (prefill)", t_pool, T * G * hd * 2 * 2.0 * (1 + 2.0 / pool), "rot_prep (Resevik attention)", t_like,
        T * (2 * H + 3 * G) * hd * 2.0, "bytes")
    # ---- decode attention
    nbd = (ctx + 16) // 16
    btd = i32(np.arange(B * nbd).reshape(B, nbd) % (nblk - 1) + 1)
    lens = i32(np.full(B, ctx))
    outd = torch.empty(B, H * hd, device=dev, dtype=bf)
    pB = proj[:B]
    splits = ops.attn_decode_splits(B, G, ctx + 16)
    ws = ops.attn_decode_workspace(B, H, hd, splits, dev)
    t_new = _time(lambda: ops.paged_attn_decode(pB, Wp, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=splits,
                                                workspace=ws, gate=pB[:, gate_col:], gate_per_head=True), flush)
    pvB, gB = projv[:B], projv[:B, gate_col:]
    t_like_d = _time(lambda: ops.paged_attn_decode(pvB, Wv, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=splits,
                                                   workspace=ws, sink=sink, gate=gB), flush)
    kvb = B * ctx * G * hd * 2 * 2.0
    put("attention decode, head gate", t_new, kvb, "attention decode, sink + gate tc", t_like_d, kvb, "bytes")
    t_gen = _time(lambda: ops.attn_sink_decode(pB, -1, kc, vc, btd, lens, None, outd, H, G, hd, hd, hd ** -0.5, window=win,
                                               head_scale=temp, pool=(pk, pv, pool)), flush)
    sp_w = ops.attn_decode_splits(B, G, min(ctx + 16, win))
    ws_w = ops.attn_decode_workspace(B, H, hd, sp_w, dev)
    prB = projr[:B]
    lse_d = torch.empty(B, H, device=dev)

    def window_then_pooled_rows():
        ops.paged_attn_decode(pB, Wp, kc, vc, btd, lens, outd, H, G, hd, hd ** -0.5, num_splits=sp_w, workspace=ws_w, window=win,
                              lse_out=lse_d)
        ops.attn_sink_decode_more(pB, kc, btd, lens, outd, lse_d, H, G, hd, hd, hd ** -0.5, win, None, (pk, pv, pool))

    t_new = _time(window_then_pooled_rows, flush)
    t_like_w = _time(lambda: ops.paged_attn_decode(prB, projr.shape[1], kc, kc, btd, lens, outd, H, G, hd, hd ** -0.5,
                                                   num_splits=sp_w, workspace=ws_w, window=win), flush)
    kvw = B * min(ctx, win) * G * hd * 2 * 2.0
    kvp = kvw + B * max(0, (ctx - win) // pool) * G * hd * 2 * 4.0
    put("attention decode, window + pooled", t_new, kvp, "attention decode, window tc", t_like_w, kvw, "bytes")
    put("attention decode, window + pooled (generic kernel alone)", t_gen, kvp, "attention decode, window tc", t_like_w, kvw,
        "bytes")

    # ---- gated diagonal recurrence (conv + gate projections + scan) vs the decayed linear attention's closing kernel
    Wd = D
    pr = rnd(T, 2 * Wd, sc=0.5)
    rb = rnd(2 * Wd, dt=f32, sc=0.1)
    cwr, cbr = rnd(Wd, conv, dt=f32, sc=0.4), rnd(Wd, dt=f32, sc=0.1)
    ringr = torch.zeros(max(S, B), conv - 1, Wd, device=dev)
    u = torch.empty(T, Wd, device=dev)
    gw = rnd(2 * H, Wd // H, Wd // H, sc=(Wd // H) ** -0.5)
    gates = torch.empty(T, 2 * Wd, device=dev)
    gb, lam = rnd(2 * Wd, dt=f32, sc=0.3), rnd(Wd, dt=f32)
    Sr = torch.zeros(max(S, B), Wd, device=dev)
    outr = torch.empty(T, Wd, device=dev, dtype=bf)
    n = Wd // H
    t_conv = _time(lambda: ops.causal_conv(pr[:, Wd:], cwr, ringr, cu, ctx0, slot_s, u, add_input=False, in_bias=rb[Wd:], bias=cbr),
                   flush)

    def gates_():
        ops.head_linear(u, gw[:H], gates[:, :Wd], H, n=n, k=n, x_head=n, out_head=n)
        ops.head_linear(u, gw[H:], gates[:, Wd:], H, n=n, k=n, x_head=n, out_head=n)

    t_gates = _time(gates_, flush)
    rws = ops.gated_recurrence_workspace(T, max(S, B), Wd, dev)
    t_scan = _time(lambda: ops.gated_recurrence_scan(u, gates, gb, lam, pr, 0, rb[:Wd], cu, ctx0, slot_s, Sr, outr, 8.0, max_len=L,
                                                     workspace=rws), flush)
    o_raw = rnd(T, Hm * hd, dt=f32)
    pl = rnd(T, 4 * Hm * hd, sc=0.5)
    mo = torch.empty(T, Hm * hd, device=dev, dtype=bf)
    t_out = _time(lambda: ops.linattn_out(o_raw, pl, 3 * Hm * hd, None, mo, Hm, hd, 1e-5, False, "silu"), flush)
    put("recurrence: causal_conv", t_conv, T * Wd * 6.0, "linattn_out (per head)", t_out, T * Hm * hd * 8.0, "bytes")
    put("recurrence: gate projections (fp32)", t_gates, T * Wd * 12.0, "linattn_out (per head)", t_out, T * Hm * hd * 8.0, "bytes")
    put("recurrence: scan (prefill)", t_scan, T * Wd * 16.0, "linattn_out (per head)", t_out, T * Hm * hd * 8.0, "bytes")
    uB, gB_, prB_, outB = u[:B], gates[:B], pr[:B], outr[:B]
    t_scan_d = _time(lambda: ops.gated_recurrence_scan(uB, gB_, gb, lam, prB_, 0, rb[:Wd], cud, ctxd, slot_b, Sr, outB, 8.0), flush)
    put("recurrence: scan (decode)", t_scan_d, B * Wd * 24.0, "linattn_out (per head)", t_out, T * Hm * hd * 8.0, "bytes")

    # ---- gated linear attention vs decayed linear attention (fixed decay per head) at equal head shapes
    xg = rnd(T, 2 * Hm * dkg + Hm * hd, dt=f32, sc=0.5)
    z = rnd(T, Hm * dkg, dt=f32, sc=2.0) + 2.0
    Sg = torch.zeros(max(S, B), Hm, hd, dkg, device=dev)
    og = torch.empty(T, Hm * hd, device=dev)
    decay = torch.tensor([0.97] * Hm, dtype=f32, device=dev)
    t_new = _time(lambda: ops.gla_scan(xg, 0, Hm * dkg, 2 * Hm * dkg, z, 1.0 / 16, cu, ctx0, slot_s, Sg, og, Hm, dkg, hd, max_len=L), flush,
                  iters=3, warm=1)
    t_like = _time(lambda: ops.linattn_scan(xg, 0, Hm * dkg, 2 * Hm * dkg, decay, cu, ctx0, slot_s, Sg, og, Hm, dkg, hd, max_len=L),
                   flush)
    wl = 4.0 * T * Hm * dkg * hd
    put("gla_scan (prefill)", t_new, wl, "linattn_scan (prefill, chunk)", t_like, wl, "flops")
    xB, zB, oB = xg[:B], z[:B], og[:B]
    t_new = _time(lambda: ops.gla_scan(xB, 0, Hm * dkg, 2 * Hm * dkg, zB, 1.0 / 16, cud, ctxd, slot_b, Sg, oB, Hm, dkg, hd, max_len=1), flush)
    t_like = _time(lambda: ops.linattn_scan(xB, 0, Hm * dkg, 2 * Hm * dkg, decay, cud, ctxd, slot_b, Sg, oB, Hm, dkg, hd, max_len=1),
                   flush)
    put("gla_scan (decode)", t_new, B * Hm * dkg * hd * 8.0, "linattn_scan (decode)", t_like, B * Hm * dkg * hd * 8.0, "bytes")
    return res


FAMILIES = {"vodavik": (vodavik_config, _kernel_numbers), "danipel": (danipel_config, _kernel_numbers_danipel),
            "resevik": (resevik_config, _kernel_numbers_resevik), "dotorax": (dotorax_config, _kernel_numbers_dotorax)}
# a family whose closest existing model is another layer-list design is measured beside that one too
CLOSEST = {"resevik": ("vodavik", vodavik_config), "dotorax": ("resevik", resevik_config)}


def run(sizes=("2k", "4k"), seqs=4, prompt=2048, batch=64, decode_steps=32, log=None, family="vodavik"):
    log = log or (lambda m: print(m, file=sys.stderr, flush=True))
    hbm, fl, how = _peaks()
    make, kernels = FAMILIES[family]
    out = {"bench": "family", "family": family, "dtype": "bf16", "data": "synthetic", "peaks": how,
           "workload": {"prefill": f"{seqs} x {prompt}", "decode": f"{batch} rows at context {prompt}", "layers": 4}, "sizes": {}}
    for size in sizes:
        log(f"size {size}: {SIZES[size]}")
        o = {"model": {}, "kernels": {}}
        models = [(family, make(size)), ("llama", llama_config(size))]
        if family in CLOSEST:
            models.insert(1, (CLOSEST[family][0], CLOSEST[family][1](size)))
        for name, cfg in models:
            o["model"][name] = _model_numbers(cfg, seqs, prompt, batch, decode_steps, log)
        o["kernels"] = kernels(size, seqs * prompt, batch, prompt, log)
        out["sizes"][size] = o
    return out
