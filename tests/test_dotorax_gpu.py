"""Dotorax (layer-list decoder: a norm before and after every sublayer, input convolutions, learned positions,
rotary attention with one gate per head, sliding-window attention with pooled blocks beside a gated diagonal
recurrence, gated linear attention) on the GPU against the plain restatement in oracle/dotorax_oracle.py.

Every test builds its own small configuration and random weights.  Kernel tests compare one mechanism with the
oracle's function; engine tests drive LLMEngine (scheduler pools, state slots, runner step functions, CUDA graphs)
and compare logits with the oracle's whole-sequence forward.  float32 must agree to rounding, bfloat16 to bf16
rounding."""
import numpy as np
import pytest
import torch

from oracle import dotorax_oracle as O

pytestmark = pytest.mark.gpu

F64 = torch.float64
BF = torch.bfloat16


def _attn(heads, kv_heads, dim, vdim, dims, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
         "rot": {"base": base, "dims": dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _par(heads, kv_heads, dim, vdim, dims, window, pool, width, blocks, conv, ls=0.6, rs=0.9, base=10000.0, scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
            "rot": {"base": base, "dims": dims}, "mask": {"size": window, "pool": pool}}
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
                                          "left_scale": ls, "right_scale": rs}}


def _gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def _ff(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def cfg_odd():
    """Nothing is a multiple of 8: every product takes the CUDA-core path.  A gla layer first; key and value widths
    that differ; rotations over part of the head; a layer without feed-forward; windows of 7 and 1 with pools of 3 and
    1; a pool larger than a page; one key head for all query heads and one per query head; two layers that read
    another layer's keys and values; four taps."""
    return {"architecture": "Dotorax", "vocab": 131, "width": 52, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "canon": {"taps": 4}, "max_positions": 700,
            "layers": [dict(_gla(3, 10, 14, 3.0), mlp=_ff(18, 1.5)),
                       dict(_par(3, 1, 10, 6, 6, 7, 3, 21, 3, 2, ls=0.4, rs=1.3, base=50.0, scale=0.9), mlp=None),
                       dict(_attn(4, 2, 6, 10, 4, base=300.0, scale=0.4), mlp=_ff(30)),
                       dict(_attn(4, 2, 6, 10, 4, base=300.0, scale=0.4, kv_from=2), mlp=_ff(22, 0.8)),
                       dict(_par(2, 2, 14, 14, 14, 1, 1, 10, 1, 1), mlp=_ff(10)),
                       dict(_par(2, 1, 12, 8, 2, 20, 19, 12, 2, 5, base=1e6), mlp=_ff(12)),
                       dict(_attn(4, 2, 6, 10, 4, base=300.0, scale=0.4, kv_from=2), mlp=None)]}


def cfg_tiles():
    """Widths that the tensor-core GEMMs take in bf16, 64-wide heads, a window of 24 with pools of 5 that prompts and
    decoding pass, two taps, a long convolution in the recurrent branch."""
    return {"architecture": "Dotorax", "vocab": 256, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 0.3,
            "canon": {"taps": 2}, "max_positions": 512,
            "layers": [dict(_attn(4, 2, 64, 64, 16, base=3e5, scale=0.11), mlp=_ff(128)),
                       dict(_par(4, 1, 64, 64, 32, 24, 5, 128, 2, 4), mlp=_ff(256, 3.0)),
                       dict(_gla(2, 64, 128, 8.0), mlp=_ff(128)),
                       dict(_attn(4, 2, 64, 64, 16, base=3e5, scale=0.11, kv_from=0), mlp=_ff(64))]}


def cfg_plain():
    """Values a model may happen to make trivial: one tap (no convolution state), a residual factor of 1, one head,
    a window longer than every sequence, mixing factors of 1, one block, one tap in the recurrent branch, tau 1, a
    full rotation, a pool of one token."""
    return {"architecture": "Dotorax", "vocab": 77, "width": 40, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
            "canon": {"taps": 1}, "max_positions": 512,
            "layers": [dict(_par(1, 1, 8, 8, 8, 4096, 4, 8, 1, 1, ls=1.0, rs=1.0), mlp=_ff(16)),
                       dict(_gla(1, 8, 8, 1.0), mlp=None),
                       dict(_attn(1, 1, 8, 8, 8), mlp=_ff(24)),
                       dict(_par(2, 2, 16, 4, 4, 3, 1, 16, 4, 2), mlp=_ff(24))]}


def cfg_wide():
    """128-wide heads in groups of four: in bf16 the attention layers (one of them on another layer's keys and values)
    run on the tcgen05 prefill and split-KV decode kernels with their one gate per head."""
    return {"architecture": "Dotorax", "vocab": 256, "width": 256, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "canon": {"taps": 3}, "max_positions": 512,
            "layers": [dict(_attn(8, 2, 128, 128, 32, base=5e5), mlp=_ff(128)),
                       dict(_par(4, 1, 128, 128, 64, 40, 8, 256, 4, 3), mlp=_ff(128)),
                       dict(_attn(8, 2, 128, 128, 32, base=5e5, kv_from=0), mlp=_ff(128))]}


CFGS = {"odd": cfg_odd, "tiles": cfg_tiles, "plain": cfg_plain, "wide": cfg_wide}


def _engine(cfg, weights, dtype, blocks=64, seqs=4, mbt=256, eager=False, max_len=512):
    from gpustack_b200.config import EngineConfig, LayerListConfig
    from gpustack_b200.engine import LLMEngine

    ecfg = EngineConfig(dtype=dtype, max_model_len=max_len, max_num_seqs=seqs, max_num_batched_tokens=mbt, num_gpu_blocks=blocks,
                        enable_prefix_caching=False, max_logit_rows=mbt, enforce_eager=eager)
    return LLMEngine.from_engine_config(ecfg, mcfg=LayerListConfig.from_dict(cfg), state_dict={k: v.cuda() for k, v in weights.items()})


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _rel(got, want):
    want = want.to(torch.float64).numpy() if isinstance(want, torch.Tensor) else want
    got = got.detach().to(torch.float64).cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    return float(np.abs(got - want).max() / max(1e-9, np.abs(want).max()))


TOL = {"float32": 3e-5, "bfloat16": 4e-2}
KTOL = {torch.float32: 2e-5, BF: 2e-2}


def _rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------------------------ mechanisms, one at a time
@pytest.mark.parametrize("D", [37, 64, 200])
@pytest.mark.parametrize("hdt", [torch.float32, BF])
def test_join_norms_the_output_before_the_sum_and_the_sum_for_the_next_sublayer(D, hdt):
    from gpustack_b200 import ops

    T, eps, m = 9, 1e-5, 0.3
    x, y, y2 = _rnd(T, D, seed=1), _rnd(T, D, seed=2, scale=3.0), _rnd(T, D, seed=3)
    wb, wa = _rnd(D, seed=4, dtype=BF, scale=0.3), _rnd(D, seed=5, dtype=BF, scale=0.3)
    for second in (False, True):
        v = (0.6 * y + 0.9 * y2) if second else y
        z = x.to(F64) + m * O.zero_centred_rms_norm(v.to(F64), wb.to(F64), eps)
        h = O.zero_centred_rms_norm(z, wa.to(F64), eps)
        xo, ho = torch.zeros(T, D, device="cuda"), torch.zeros(T, D, dtype=hdt, device="cuda")
        ops.sandwich_join(x.cuda(), eps, y=y.cuda(), y2=y2.cuda() if second else None, ya=0.6 if second else 1.0, yb=0.9,
                          post_w=wb.cuda(), mult=m, pre_w=wa.cuda(), x_out=xo, h_out=ho)
        assert _rel(xo, z) < 2e-6
        assert _rel(ho, h) < (2e-6 if hdt == torch.float32 else 8e-3)
    # no output yet (the first sublayer), in place, and the gather of chosen rows
    xc = x.cuda().clone()
    ho = torch.zeros(T, D, device="cuda")
    ops.sandwich_join(xc, eps, pre_w=wa.cuda(), h_out=ho)
    assert _rel(ho, O.zero_centred_rms_norm(x.to(F64), wa.to(F64), eps)) < 2e-6
    ops.sandwich_join(xc, eps, y=y.cuda(), post_w=wb.cuda(), mult=m, x_out=xc)
    z = x.to(F64) + m * O.zero_centred_rms_norm(y.to(F64), wb.to(F64), eps)
    assert _rel(xc, z) < 2e-6
    rows = [7, 0, 3]
    hg = torch.zeros(3, D, dtype=hdt, device="cuda")
    ops.sandwich_join(x.cuda(), eps, y=y.cuda(), post_w=wb.cuda(), mult=m, pre_w=wa.cuda(), rows=_i32(rows), h_out=hg)
    assert _rel(hg, O.zero_centred_rms_norm(z, wa.to(F64), eps)[rows]) < (2e-6 if hdt == torch.float32 else 8e-3)


def test_embedding_plus_learned_position():
    from gpustack_b200 import ops

    table, pos = _rnd(50, 24, seed=1, dtype=BF), _rnd(90, 24, seed=2, dtype=BF)
    ids, p = [3, 49, 0, 7], [0, 89, 17, 17]
    x = torch.zeros(4, 24, device="cuda")
    ops.embed_pos(_i32(ids), _i32(p), table.cuda(), pos.cuda(), x)
    assert torch.equal(x.cpu(), table[ids].float() + pos[p].float())


@pytest.mark.parametrize("taps", [1, 2, 3, 4])
@pytest.mark.parametrize("C", [21, 64])
@pytest.mark.parametrize("residual", [True, False])
def test_short_convolution_in_portions_with_rings_that_are_used_again(taps, C, residual):
    """Two sequences in two ring slots, cut into portions of 1 .. 9 rows that ride in the same launches; then a third
    sequence takes the first one's slot without any clearing.  Each equals the convolution of the whole sequence."""
    from gpustack_b200 import ops

    w = _rnd(C, taps, seed=1, scale=0.5)
    bias, in_bias = (None, None) if residual else (_rnd(C, seed=2), _rnd(C, seed=3))
    seqs = {"a": _rnd(37, C, seed=4), "b": _rnd(22, C, seed=5), "c": _rnd(15, C, seed=6)}
    want = {}
    for k, x in seqs.items():
        xin = x.to(F64) + (0 if in_bias is None else in_bias.to(F64))
        want[k] = O.causal_conv(xin, w.to(F64), None if bias is None else bias.to(F64)) + (xin if residual else 0)
    ring = torch.full((2, max(taps - 1, 1), C), 7.0, device="cuda")[:, :taps - 1] if taps > 1 else None
    if ring is not None:
        ring = ring.contiguous()
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}
    slot = {"a": 1, "b": 0, "c": 1}
    plan = [[("a", 9), ("b", 1)], [("a", 1), ("b", 2)], [("a", 2), ("b", 1)], [("b", 5), ("a", 3)], [("a", 22), ("b", 13)],
            [("c", 1)], [("c", 1)], [("c", 2)], [("c", 11)]]
    for step in plan:
        rows = torch.cat([seqs[k][at[k]:at[k] + n] for k, n in step]).cuda().contiguous()
        cu = np.cumsum([0] + [n for _, n in step]).tolist()
        out = torch.zeros_like(rows)
        args = (_i32(cu), _i32([at[k] for k, _ in step]), _i32([slot[k] for k, _ in step]))
        kw = dict(in_bias=None if in_bias is None else in_bias.cuda())
        ops.causal_conv(rows, w.cuda(), ring, *args, out, add_input=residual, bias=None if bias is None else bias.cuda(), **kw)
        if ring is not None:
            ops.conv_commit(rows, ring, *args, taps, **kw)
        for (k, n), lo in zip(step, cu):
            got[k].append(out[lo:lo + n].cpu())
            at[k] += n
    for k in seqs:
        assert at[k] == len(seqs[k])
        assert _rel(torch.cat(got[k]), want[k]) < 2e-6, k


def _paged(k, v, dtype, seed, extra=3, page=16):
    """Keys / values [n, G, w] in shuffled pages (junk elsewhere)."""
    n, G = k.shape[0], k.shape[1]
    nb = (n + page - 1) // page
    perm = torch.randperm(nb + extra, generator=torch.Generator().manual_seed(seed))[:nb]
    kc = torch.full((nb + extra, G, page, k.shape[2]), 50.0, dtype=dtype)
    vc = torch.full((nb + extra, G, page, v.shape[2]), -50.0, dtype=dtype)
    for t in range(n):
        kc[perm[t // page], :, t % page] = k[t]
        vc[perm[t // page], :, t % page] = v[t]
    return kc.cuda(), vc.cuda(), perm.to(torch.int32)


def _pool_case(dtype, n, H, G, dk, dv, seed, stand=None):
    """q / k / v of one sequence; stand = (i, js): the keys js are aligned with query i's first head of every group and
    made large, their values 10 -- so that they (or the mean of their block) take query i's whole softmax if seen."""
    q, k, v = _rnd(n, H, dk, seed=seed), _rnd(n, G, dk, seed=seed + 1), _rnd(n, G, dv, seed=seed + 2)
    if stand is not None:
        i, js = stand
        for g in range(G):
            for j in js:
                k[j, g] = 8.0 * q[i, g * (H // G)] / q[i, g * (H // G)].norm() * dk ** 0.5
                v[j, g] = 10.0
    return q.to(dtype), k.to(dtype), v.to(dtype)


def _run_pooled(q, k, v, H, G, window, pool, scale, head_scale, cuts, seed=3):
    """The sequence through the cache in portions `cuts` (a portion of one row with context runs through the decode
    kernel): block means refreshed, then attention.  -> outputs of all rows."""
    from gpustack_b200 import ops

    dtype = q.dtype
    n, dk, dv = q.shape[0], q.shape[2], v.shape[2]
    kc, vc, perm = _paged(k, v, dtype, seed)
    per_page = -(-16 // pool)
    pk = torch.full((kc.shape[0], G, per_page, dk), 99.0, device="cuda")
    pv = torch.full((kc.shape[0], G, per_page, dv), -99.0, device="cuda")
    bt = perm.cuda().reshape(1, -1)
    hs = None if head_scale is None else head_scale.float().cuda()
    outs, at = [], 0
    for c in cuts:
        rows = q[at:at + c].reshape(c, H * dk).cuda().contiguous()
        out = torch.zeros(c, H * dv, dtype=dtype, device="cuda")
        if c == 1 and at > 0:
            ops.kv_pool_update(kc, vc, pk, pv, bt, None, _i32([at + 1]), 1, 1, pool)
            ops.attn_sink_decode(rows, -1, kc, vc, bt, _i32([at + 1]), None, out, H, G, dk, dv, scale, window=window,
                                 head_scale=hs, pool=(pk, pv, pool))
        else:
            ops.kv_pool_update(kc, vc, pk, pv, bt, _i32([0, c]), _i32([at]), 1, c, pool)
            ts, tq = ops.build_prefill_tiles([c], ops.attn_sink_prefill_tile(), [at])
            ops.attn_sink_prefill(rows, -1, kc, vc, bt, _i32([0, c]), _i32([at]), _i32(ts), _i32(tq), None, out, H, G, dk, dv,
                                  scale, window=window, head_scale=hs, pool=(pk, pv, pool))
        outs.append(out.cpu())
        at += c
    assert at == n
    return torch.cat(outs)


def _cuts(n, sizes):
    out, i = [], 0
    while sum(out) < n:
        out.append(min(sizes[i % len(sizes)], n - sum(out)))
        i += 1
    return out


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("H,G,dk,dv,window,pool,n", [(3, 1, 10, 6, 7, 3, 90), (4, 2, 64, 64, 24, 5, 150), (2, 2, 14, 14, 1, 1, 50),
                                                      (2, 1, 12, 8, 20, 19, 140), (6, 1, 32, 16, 40, 16, 200), (2, 1, 8, 8, 500, 4, 70),
                                                      (4, 4, 16, 24, 33, 12, 130)])
def test_window_with_pooled_blocks_in_portions_over_shuffled_pages(dtype, H, G, dk, dv, window, pool, n):
    """Whole, token by token, and in portions down to two rows: cuts inside blocks, pages and the window."""
    scale = 0.3
    temp = 1.0 + 0.3 * _rnd(H, seed=9)
    q, k, v = _pool_case(dtype, n, H, G, dk, dv, seed=21)
    want = O.pooled_window_attention(q.to(F64), k.to(F64), v.to(F64), scale * temp.to(F64), window, pool).reshape(n, -1)
    for cuts in ([n], [1] * n, _cuts(n, [2, 3, 11, 16, 2, 17, 1, 5, 31, 1, 1, 2])):
        got = _run_pooled(q, k, v, H, G, window, pool, scale, temp, cuts)
        assert _rel(got, want) < KTOL[dtype], cuts[:4]


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("window,pool,i", [(7, 3, 60), (16, 4, 47), (17, 16, 64), (24, 5, 98), (33, 12, 80), (1, 1, 20), (20, 19, 95),
                                           (40, 7, 130)])
@pytest.mark.parametrize("what", ["window_in", "window_out", "pool_in", "pool_out"])
def test_keys_at_the_edges_of_the_window_and_of_the_pooled_blocks(dtype, window, pool, i, what):
    """window_in: key i - window + 1, the last token query i sees, made large -- it takes the softmax.  window_out: key
    i - window, not seen as a token (and its block is seen only if it ends there).  pool_in: the whole block that ends
    at or just before i - window made large -- its mean takes the softmax.  pool_out: the block after it, which still
    reaches into the window: its tokens outside the window are seen neither as tokens nor through a mean.  Prompt rows
    (portions that start before and at the query) and the decode kernel."""
    H, G, dk, dv, scale = 2, 1, 16, 16, 1.0
    last_seen = (i - window + 1) // pool - 1            # the newest block query i sees
    if what == "window_in":
        js = [i - window + 1]
    elif what == "window_out":
        js = [i - window]
    elif what == "pool_in":
        js = list(range(last_seen * pool, last_seen * pool + pool))
    else:
        js = [j for j in range((last_seen + 1) * pool, (last_seen + 2) * pool) if j <= i - window]
    if not js or min(js) < 0:
        pytest.skip("no such key for these sizes")
    n = i + 1
    q, k, v = _pool_case(dtype, n, H, G, dk, dv, seed=13, stand=(i, js))
    want = O.pooled_window_attention(q.to(F64), k.to(F64), v.to(F64), torch.full((H,), scale, dtype=F64), window, pool).reshape(n, -1)
    seen = float(want[i, :dv].min()) > 9.0              # head 0 is the one the keys were aligned with
    if what in ("window_in", "pool_in"):
        assert seen
    elif what == "pool_out" or (i - window + 1) % pool != 0:
        assert not seen                                 # (a window_out key that closes a block is seen through its mean)
    for cuts in ([n], [i, 1], [max(1, min(js)), n - max(1, min(js))], [n - 2, 2], [i - 1, 1, 1]):
        cuts = [c for c in cuts if c > 0]
        if sum(cuts) != n:
            continue
        got = _run_pooled(q, k, v, H, G, window, pool, scale, None, cuts)
        assert _rel(got[i:], want[i:]) < KTOL[dtype], (what, cuts)
        assert _rel(got, want) < KTOL[dtype], (what, cuts)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("H,G,dk,dv,dims", [(4, 2, 6, 10, 4), (4, 2, 64, 64, 16), (1, 1, 8, 8, 8), (6, 3, 24, 40, 12)])
def test_rotated_attention_with_one_gate_per_head_and_queries_only_for_a_borrowed_cache(dtype, H, G, dk, dv, dims):
    """Projection rows [q | k | v | gate (H columns)]: rotation (half-split) of q and k, keys and values to their
    pages; then a second mixer with rows [q | gate] that prepares only its queries and reads the same pages."""
    from gpustack_b200 import ops

    n, scale, base = 45, 0.4, 300.0
    pos = torch.arange(n)
    qw, gw = H * dk, H
    raw = _rnd(n, qw + G * dk + G * dv + gw, seed=5).to(dtype)
    raw2 = _rnd(n, qw + gw, seed=6).to(dtype)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).cuda()
    k = O.rotate(raw[:, qw:qw + G * dk].to(F64).reshape(n, G, dk), pos, base, dims, "half")
    v = raw[:, qw + G * dk:qw + G * (dk + dv)].to(F64).reshape(n, G, dv)
    if dtype == BF:
        k = k.to(BF).to(F64)
    nb = (n + 15) // 16
    kc = torch.zeros(nb + 1, G, 16, dk, dtype=dtype, device="cuda")
    vc = torch.zeros(nb + 1, G, 16, dv, dtype=dtype, device="cuda")
    bt = torch.arange(1, nb + 1, dtype=torch.int32, device="cuda").reshape(1, -1)
    slots = _i32([16 + t for t in range(n)])
    ts, tq = ops.build_prefill_tiles([n], ops.attn_sink_prefill_tile(), [0])
    for rows, own in ((raw, True), (raw2, False)):
        proj = rows.cuda().clone()
        ops.rot_prep(proj, 0, qw, qw + G * dk, _i32(list(range(n))), slots, proj, kc if own else None, vc if own else None,
                     H, G, dk, dv, paged=True, rot_dims=dims, half_layout=True, freq=freq)
        qr = O.rotate(rows[:, :qw].to(F64).reshape(n, H, dk), pos, base, dims, "half")
        assert _rel(proj[:, :qw], qr.reshape(n, -1)) < KTOL[dtype]
        if not own:
            assert torch.equal(proj[:, qw:].cpu(), rows[:, qw:])
        if dtype == BF:
            qr = qr.to(BF).to(F64)
        gate_col = qw + (G * (dk + dv) if own else 0)
        out = torch.zeros(n, H * dv, dtype=dtype, device="cuda")
        ops.attn_sink_prefill(proj, gate_col, kc, vc, bt, _i32([0, n]), _i32([0]), _i32(ts), _i32(tq), None, out, H, G, dk, dv,
                              scale, gate_per_head=True)
        want = O.causal_attention(qr, k, v, scale) * torch.sigmoid(rows[:, gate_col:gate_col + H].to(F64)).unsqueeze(-1)
        assert _rel(out, want.reshape(n, -1)) < KTOL[dtype]
        od = torch.zeros(1, H * dv, dtype=dtype, device="cuda")
        ops.attn_sink_decode(proj[n - 1:], gate_col, kc, vc, bt, _i32([n]), None, od, H, G, dk, dv, scale, gate_per_head=True)
        assert _rel(od, want.reshape(n, -1)[n - 1:]) < KTOL[dtype]


@pytest.mark.parametrize("H,G,dk,n,start,splits", [(8, 2, 128, 200, 0, 1), (8, 1, 128, 150, 37, 3), (4, 2, 64, 90, 0, 2)])
def test_one_gate_per_head_on_the_tensor_core_attention_kernels(H, G, dk, n, start, splits):
    """bf16, tile-sized heads: the tcgen05 prefill kernel (128-wide heads in groups of four and eight) and the split-KV
    decode kernel multiply a head's output by sigmoid of the head's ONE gate column."""
    from gpustack_b200 import ops

    scale = 0.09
    q, k, v = _pool_case(BF, n, H, G, dk, dk, seed=31)
    gate = _rnd(n, 8, seed=32, scale=2.0).to(BF)           # H gate columns, padded to 16-byte rows
    want = (O.causal_attention(q.to(F64), k.to(F64), v.to(F64), scale) * torch.sigmoid(gate[:, :H].to(F64)).unsqueeze(-1)).reshape(n, -1)
    kc, vc, perm = _paged(k, v, BF, 5)
    bt = perm.cuda().reshape(1, -1)
    rows = torch.cat([q.reshape(n, H * dk), gate], dim=1)[start:].cuda().contiguous()      # [q | gate columns]
    if ops.attn_prefill_tc_covers(H, G, dk):
        out = torch.zeros(n - start, H * dk, dtype=BF, device="cuda")
        ts, tq = ops.build_prefill_tiles([n - start], ops.attn_prefill_tile(H, G), [start])
        ops.paged_attn_prefill_ex(rows, rows.stride(0), kc, vc, bt, _i32([0, n - start]), _i32([start]), _i32(ts), _i32(tq), out,
                                  H, G, dk, scale, gate=rows[:, H * dk:], gate_per_head=True)
        assert _rel(out, want[start:]) < KTOL[BF]
    last = rows[-1:]
    od = torch.zeros(1, H * dk, dtype=BF, device="cuda")
    ws = ops.attn_decode_workspace(1, H, dk, splits, "cuda")
    ops.paged_attn_decode(last, last.stride(0), kc, vc, bt, _i32([n]), od, H, G, dk, scale, num_splits=splits, workspace=ws,
                          gate=last[:, H * dk:], gate_per_head=True)
    assert _rel(od, want[n - 1:]) < KTOL[BF]


@pytest.mark.parametrize("H,G,dk,window,pool,n,start", [(8, 2, 128, 40, 8, 300, 0), (4, 1, 128, 64, 5, 260, 33),
                                                         (8, 1, 128, 24, 16, 200, 128), (8, 2, 128, 500, 4, 150, 0),
                                                         (3, 1, 128, 33, 7, 231, 0), (12, 2, 64, 16, 3, 177, 0)])
def test_window_on_the_tensor_cores_continued_over_the_pooled_blocks(H, G, dk, window, pool, n, start):
    """bf16, tile-sized heads: the tcgen05 prefill kernel (128-wide heads in groups of four and eight) and the split-KV
    decode kernel attend the window's tokens and hand over every row's log-sum-exp; the generic kernels continue that
    softmax over the pooled blocks.  The per-head temperature rides in the queries."""
    from gpustack_b200 import ops

    scale = 0.09
    temp = 1.0 + 0.3 * _rnd(H, seed=9)
    q, k, v = _pool_case(BF, n, H, G, dk, dk, seed=41)
    want = O.pooled_window_attention(q.to(F64), k.to(F64), v.to(F64), scale * temp.to(F64), window, pool).reshape(n, -1)
    kc, vc, perm = _paged(k, v, BF, 7)
    pk = torch.zeros(kc.shape[0], G, -(-16 // pool), dk, device="cuda")
    pv = torch.zeros_like(pk)
    bt = perm.cuda().reshape(1, -1)
    ops.kv_pool_update(kc, vc, pk, pv, bt, _i32([0, n]), _i32([0]), 1, n, pool)
    rows = (q.float() * temp.reshape(1, H, 1)).to(BF)[start:].reshape(n - start, H * dk).cuda().contiguous()
    out = torch.zeros_like(rows)
    lse = torch.zeros(n - start, H, device="cuda")
    if ops.attn_prefill_tc_covers(H, G, dk):
        tile = ops.attn_prefill_tile(H, G)
        ts, tq = ops.build_prefill_tiles([n - start], tile, [start])
        args = (bt, _i32([0, n - start]), _i32([start]), _i32(ts), _i32(tq))
        ops.paged_attn_prefill_ex(rows, rows.stride(0), kc, vc, *args, out, H, G, dk, scale, window=window, lse_out=lse)
        ops.attn_sink_prefill_more(rows, kc, *args, out, lse, H, G, dk, dk, scale, tile, window, None, (pk, pv, pool))
        assert _rel(out, want[start:]) < KTOL[BF]
    # single rows at several lengths (a pooled block that has just come into sight and one that has not yet), whole
    # key range and split
    for m in sorted({n, n - 1, window + pool - 1, window + pool, window + 2 * pool, max(1, window - 1)}):
        if not start < m <= n:
            continue
        last = rows[m - 1 - start:m - start]
        for splits in (1, 3):
            od, lse1 = torch.zeros(1, H * dk, dtype=BF, device="cuda"), torch.zeros(1, H, device="cuda")
            ws = ops.attn_decode_workspace(1, H, dk, splits, "cuda")
            ops.paged_attn_decode(last, last.stride(0), kc, vc, bt, _i32([m]), od, H, G, dk, scale, num_splits=splits,
                                  workspace=ws, window=window, lse_out=lse1)
            ops.attn_sink_decode_more(last, kc, bt, _i32([m]), od, lse1, H, G, dk, dk, scale, window, None, (pk, pv, pool))
            assert _rel(od, want[m - 1:m]) < KTOL[BF], (m, splits)


@pytest.mark.parametrize("W,blocks", [(21, 3), (128, 2), (10, 1), (96, 12)])
@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_gated_diagonal_recurrence_in_portions_and_a_slot_that_is_used_again(W, blocks, dtype):
    from gpustack_b200 import ops

    n = W // blocks
    w = {"ra": _rnd(blocks, n, n, seed=1, scale=n ** -0.5), "ri": _rnd(blocks, n, n, seed=2, scale=n ** -0.5),
         "ra.b": _rnd(blocks, n, seed=3, scale=0.3), "ri.b": _rnd(blocks, n, seed=4, scale=0.3), "lam": _rnd(W, seed=5, scale=1.5) - 1.0}
    w = {k: t.to(BF).float() for k, t in w.items()}
    yb = _rnd(W, seed=6, scale=0.3)
    S = torch.full((2, W), 5.0, device="cuda")
    gates_w = torch.cat([w["ra"], w["ri"]]).to(BF).cuda()
    gate_b = torch.cat([w["ra.b"].reshape(-1), w["ri.b"].reshape(-1)]).cuda()
    for name, T, cuts in (("a", 60, [60]), ("b", 41, [3, 1, 1, 2, 17, 1, 16])):      # b takes a's slot afterwards
        u, y = _rnd(T, W, seed=7 + T), _rnd(T, W, seed=8 + T).to(dtype)
        rec = O.gated_diagonal_recurrence(u.to(F64), {k: t.to(F64) for k, t in w.items()}, blocks)
        want = rec * O.gelu_tanh(y.to(F64) + yb.to(F64))
        at, got = 0, []
        for c in cuts:
            uu = u[at:at + c].cuda().contiguous()
            g = torch.zeros(c, 2 * W, device="cuda")
            ops.head_linear(uu, gates_w[:blocks], g[:, :W], blocks, n=n, k=n, x_head=n, out_head=n)
            ops.head_linear(uu, gates_w[blocks:], g[:, W:], blocks, n=n, k=n, x_head=n, out_head=n)
            proj = torch.cat([_rnd(c, 5, seed=1).to(dtype), y[at:at + c]], dim=1).cuda().contiguous()
            out = torch.zeros(c, W, dtype=dtype, device="cuda")
            ops.gated_recurrence_scan(uu, g, gate_b, w["lam"].cuda(), proj, 5, yb.cuda(), _i32([0, c]), _i32([at]), _i32([1]), S, out, 8.0)
            got.append(out.cpu())
            at += c
        assert _rel(torch.cat(got), want) < (1e-5 if dtype == torch.float32 else 8e-3), name
        assert _rel(S[1], rec[-1]) < 1e-5


def _gla_ref(q, k, v, z, tau):
    T, H, dk = q.shape
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).reshape(T, H, dk)
    S = torch.zeros(H, dk, v.shape[2], dtype=q.dtype)
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = alpha[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


@pytest.mark.parametrize("H,dk,dv,tau", [(3, 10, 14, 3.0), (2, 64, 128, 8.0), (1, 8, 8, 1.0), (2, 33, 70, 16.0), (1, 128, 40, 2.0),
                                          (1, 200, 24, 4.0), (2, 256, 36, 5.0)])
def test_gated_linear_attention_in_portions_against_the_recurrence(H, dk, dv, tau):
    from gpustack_b200 import ops

    T = 75
    x = _rnd(T, 2 * H * dk + H * dv, seed=3, scale=0.7)
    z = _rnd(T, H * dk, seed=4, scale=2.0) + 1.0
    q, k = x[:, :H * dk].reshape(T, H, dk), x[:, H * dk:2 * H * dk].reshape(T, H, dk)
    v = x[:, 2 * H * dk:].reshape(T, H, dv)
    want, S_end = _gla_ref(q.to(F64), k.to(F64), v.to(F64), z.to(F64), tau)
    # (the bound of the new rows per sequence picks the kernel: single rows have their own; 0 = unknown)
    for cuts, bound in (([T], T), ([1] * T, 1), ([1] * T, 0), (_cuts(T, [2, 3, 16, 1, 17, 1, 5, 31]), 31)):
        S = torch.full((3, H, dv, dk), 4.0, device="cuda")
        at, got = 0, []
        for c in cuts:
            o = torch.zeros(c, H * dv, device="cuda")
            ops.gla_scan(x[at:at + c].cuda().contiguous(), 0, H * dk, 2 * H * dk, z[at:at + c].cuda().contiguous(), 1.0 / tau,
                         _i32([0, c]), _i32([at]), _i32([2]), S, o, H, dk, dv, max_len=bound)
            got.append(o.cpu())
            at += c
        assert _rel(torch.cat(got), want.reshape(T, -1)) < 2e-5
        assert _rel(S[2].transpose(1, 2), S_end) < 2e-5
        assert float(S[0].min()) == 4.0 and float(S[1].max()) == 4.0


def test_a_key_far_back_survives_a_slow_decay_and_dies_under_a_fast_one():
    """One key / value pair at position 3 and a query aligned with it at position 400: with sigmoid(z) close to one the
    state still holds the pair; with a fast decay in the key's channels nothing is left."""
    from gpustack_b200 import ops

    H, dk, dv, T = 1, 16, 8, 401
    x = torch.zeros(T, 2 * dk + dv)
    x[3, dk:2 * dk] = 1.0
    x[3, 2 * dk:] = 5.0
    x[400, :dk] = 1.0 / dk
    for zval, alive in ((12.0, True), (0.0, False)):
        z = torch.full((T, dk), zval)
        S = torch.zeros(1, H, dv, dk, device="cuda")
        o = torch.zeros(T, dv, device="cuda")
        ops.gla_scan(x.cuda(), 0, dk, 2 * dk, z.cuda(), 1.0, _i32([0, T]), _i32([0]), _i32([0]), S, o, H, dk, dv)
        want, _ = _gla_ref(x[:, :dk].reshape(T, 1, dk).to(F64), x[:, dk:2 * dk].reshape(T, 1, dk).to(F64),
                           x[:, 2 * dk:].reshape(T, 1, dv).to(F64), z.to(F64), 1.0)
        assert (float(want[400].min()) > 4.9) == alive
        assert abs(float(o[400].min()) - float(want[400].min())) < 1e-4


# ------------------------------------------------------------------------------------ whole models through the engine
def _close(got, want, dtype):
    """float32: every logit to rounding.  bfloat16: rounding noise is not uniform over positions (a narrow model with a
    residual factor of 1 and sharp decays amplifies it here and there), while a fault of the cache, the state or the
    batch moves most positions: at most one position in twenty may be off, and the typical one is well inside."""
    if dtype == "float32":
        return _rel(got, want) < TOL[dtype]
    want = want.to(torch.float64).numpy() if isinstance(want, torch.Tensor) else np.asarray(want, dtype=np.float64)
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1) / np.abs(want).max()
    return float(np.mean(err > TOL[dtype])) <= 0.05 and float(np.median(err)) < TOL[dtype] / 2


@pytest.fixture(scope="module", params=list(CFGS))
def model(request):
    cfg = CFGS[request.param]()
    return cfg, O.random_weights(cfg, seed=3 + len(request.param))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer(model, dtype):
    cfg, W = model
    toks = _tokens(cfg, 70, 1)
    trail = []
    want = O.forward(cfg, W, toks, trace=trail)
    eng = _engine(cfg, W, dtype)
    seen = eng.runner.layer_trace = []
    got = eng.replay_step([("a", toks, list(range(len(toks))))], ["a"])
    eng.runner.layer_trace = None
    assert len(seen) == len(cfg["layers"]) == len(trail)
    for l in range(len(seen)):
        assert _rel(seen[l], trail[l]) < TOL[dtype] * 2, f"residual stream after layer {l}"
    assert _close(got, want, dtype)
    # the serving path (sums folded into the next norm) gives the same logits as the traced one
    again = eng.replay_step([("b", toks, list(range(len(toks))))], ["b"])
    assert _rel(again, got) < (1e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_single_tokens_match_the_whole_prompt(model, dtype):
    """One prompt, token by token, and portions of changing size down to two tokens (page size 16, windows of 1 / 3 / 7 /
    20 / 24, pools of 1 / 3 / 5 / 19, two to four taps: cuts inside and at their borders): the logits at a position do
    not depend on the cut."""
    cfg, W = model
    toks = _tokens(cfg, 90, 2)
    want = O.forward(cfg, W, toks)
    eng = _engine(cfg, W, dtype)
    whole = eng.replay_step([("w", toks, list(range(len(toks))))], ["w"])
    one = np.concatenate([eng.replay_step([("t", toks[i:i + 1], [0])], ["t"] if i == len(toks) - 1 else []) for i in range(len(toks))])
    parts, pos, i = [], 0, 0
    sizes = [2, 3, 11, 16, 2, 17, 1, 5, 31, 2]
    while pos < len(toks):
        c = min(sizes[i % len(sizes)], len(toks) - pos)
        parts.append(eng.replay_step([("p", toks[pos:pos + c], list(range(c)))], ["p"] if pos + c == len(toks) else []))
        pos, i = pos + c, i + 1
    parts = np.concatenate(parts)
    for got in (whole, one, parts):
        assert _close(got, want, dtype)
    if dtype == "float32":
        assert _rel(one, whole) < 1e-5 and _rel(parts, whole) < 1e-5
    assert eng.sched.pool.num_free == eng.sched.pool.num_total


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests_with_reused_pages_and_slots(model, dtype):
    """Five requests of unequal length through four sequence / state slots and too few pages for all of them at once:
    portions of some ride beside single tokens of others, a finished request's pages, state slot and convolution rings
    go to the next one (whose recurrences start from zero and whose pooled blocks are written anew).  Every request's
    logits equal those of the request alone."""
    cfg, W = model
    lens = [61, 9, 120, 33, 47]
    reqs = {f"r{i}": _tokens(cfg, n, 20 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, W, t).numpy() for k, t in reqs.items()}
    eng = _engine(cfg, W, dtype, blocks=17, seqs=4)     # 16 pages: the five requests need 19, so pages are reused
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    plan = [[("r0", 30), ("r1", 2)], [("r0", 1), ("r1", 7), ("r2", 50)], [("r0", 1), ("r2", 17), ("r3", 33)],
            [("r0", 29), ("r2", 1)], [("r2", 1), ("r4", 2)], [("r2", 51), ("r4", 1)], [("r4", 1)], [("r4", 43)]]
    for step in plan:
        entries, end = [], []
        for rid, n in step:
            lo = at[rid]
            entries.append((rid, reqs[rid][lo:lo + n], list(range(n))))
            at[rid] = lo + n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        out = eng.replay_step(entries, end)
        off = 0
        for rid, n in step:
            got[rid].append(out[off:off + n])
            off += n
    assert all(at[k] == len(reqs[k]) for k in reqs)
    for k in reqs:
        assert _close(np.concatenate(got[k]), want[k], dtype), k
    assert eng.sched.pool.num_free == eng.sched.pool.num_total
    assert eng.sched.slots.num_free == 4
    assert eng.runner.stats.get("mixed_steps", 0) >= 4 and eng.runner.stats["decode_steps"] >= 1


def _random_cfg(rng):
    """A random model: layer kinds, order, head counts, widths (odd and tile-sized), windows, pools, taps, rotations and
    constants all drawn anew."""
    D = rng.choice([48, 64, 96, 128, 192, 256, 320])
    n = rng.randint(2, 6)
    layers, owners = [], []
    for l in range(n):
        kind = rng.choice(["attention", "parallel", "gla"])
        G = rng.choice([1, 2, 3, 4])
        H = G * rng.choice([1, 2, 3, 4])
        dk, dv = rng.choice([8, 16, 20, 24, 32, 64, 128]), rng.choice([8, 12, 16, 32, 40, 64, 128])
        dims = rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dk])
        if kind == "attention" and owners and rng.random() < 0.4:
            src = rng.choice(owners)
            layer = _attn(**dict(src[1], kv_from=src[0]))
        elif kind == "attention":
            kw = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, dims=dims, base=rng.choice([100.0, 1e4, 5e5]), scale=rng.choice([dk ** -0.5, 0.2]))
            layer = _attn(**kw)
            owners.append((l, kw))
        elif kind == "parallel":
            blocks = rng.choice([1, 2, 4, 5])
            layer = _par(H, G, dk, dv, dims, rng.choice([1, 2, 5, 16, 17, 33, 48, 64, 100, 1000]), rng.choice([1, 2, 3, 7, 12, 16, 20]),
                         blocks * rng.choice([4, 8, 13, 32]), blocks, rng.choice([1, 2, 4]), ls=rng.choice([0.5, 1.0, 1.4]),
                         rs=rng.choice([0.3, 1.0]), base=rng.choice([100.0, 1e4]))
        else:
            layer = _gla(rng.choice([1, 2, 3, 6]), rng.choice([8, 12, 16, 48, 64]), rng.choice([8, 12, 16, 32, 64]), rng.choice([1.0, 4.0, 16.0]))
        layers.append(dict(layer, mlp=_ff(rng.choice([16, 24, 64, 96, 128, 256]), rng.choice([0.5, 2.0, 7.0])) if rng.random() < 0.8 else None))
    return {"architecture": "Dotorax", "vocab": rng.choice([100, 257, 1000]), "width": D, "norm": {"eps": rng.choice([1e-5, 1e-6])},
            "residual_mult": rng.choice([0.2, 0.5, 1.0]), "canon": {"taps": rng.choice([1, 2, 3, 4, 5])}, "max_positions": 400,
            "layers": layers}


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106])
def test_random_configurations_in_float32(seed):
    """Whole prompt, and two requests in portions beside single tokens, against the oracle."""
    import random

    rng = random.Random(seed)
    cfg = _random_cfg(rng)
    W = O.random_weights(cfg, seed=seed, decay_rank=rng.choice([1, 4, 16]))
    t1, t2 = _tokens(cfg, 150, seed), _tokens(cfg, 70, seed + 1)
    w1, w2 = O.forward(cfg, W, t1), O.forward(cfg, W, t2)
    eng = _engine(cfg, W, "float32", blocks=20)
    assert _rel(eng.replay_step([("a", t1, list(range(150)))], ["a"]), w1) < TOL["float32"]
    toks, at, got = {"x": t1, "y": t2}, {"x": 0, "y": 0}, {"x": [], "y": []}
    for step in ([("x", 37), ("y", 2)], [("x", 2), ("y", 30)], [("x", 1), ("y", 1)], [("x", 64), ("y", 1)], [("x", 1), ("y", 36)], [("x", 45)]):
        entries, end = [], []
        for rid, n in step:
            entries.append((rid, toks[rid][at[rid]:at[rid] + n], list(range(n))))
            at[rid] += n
            if at[rid] == len(toks[rid]):
                end.append(rid)
        out, off = eng.replay_step(entries, end), 0
        for rid, n in step:
            got[rid].append(out[off:off + n])
            off += n
    assert _rel(np.concatenate(got["x"]), w1) < TOL["float32"] and _rel(np.concatenate(got["y"]), w2) < TOL["float32"]
    assert eng.sched.pool.num_free == eng.sched.pool.num_total


def test_long_decoding_through_the_graphs_in_float32():
    """300 single-token steps after a short prompt through the captured decode graphs: every window slides over decoded
    tokens many times, blocks are completed and pooled while decoding, the decode kernel walks 20 pages, the recurrent
    states and the convolution rings pass through 300 updates."""
    cfg = cfg_odd()
    W = O.random_weights(cfg, seed=5)
    toks = _tokens(cfg, 320, 9)
    want = O.forward(cfg, W, toks)
    eng = _engine(cfg, W, "float32")
    out = [eng.replay_step([("a", toks[:20], list(range(20)))], [])]
    for i in range(20, len(toks)):
        out.append(eng.replay_step([("a", toks[i:i + 1], [0])], ["a"] if i == len(toks) - 1 else []))
    assert _rel(np.concatenate(out), want) < TOL["float32"]
    assert eng.runner.stats["graph_replays"] >= 290


@pytest.mark.parametrize("name,dtype,eager", [("odd", "float32", True), ("tiles", "bfloat16", False), ("plain", "bfloat16", False)])
def test_greedy_generation_through_the_scheduler(name, dtype, eager):
    """LLMEngine.generate: continuous batching of six prompts over four sequence and state slots, chunked prefill
    (token budget 48), decode steps.  The oracle is teacher-forced on the engine's tokens; wherever its top-2 margin
    is decisive the engine's token is its argmax."""
    from gpustack_b200.scheduler import SamplingParams

    cfg = CFGS[name]()
    W = O.random_weights(cfg, seed=8)
    prompts = [_tokens(cfg, n, 40 + n) for n in (5, 70, 23, 1, 64, 17)]
    eng = _engine(cfg, W, dtype, blocks=40, seqs=4, mbt=48, eager=eager)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    tol = 1e-4 if dtype == "float32" else 3e-2
    checked = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        lg = O.forward(cfg, W, p + o)
        for t in range(12):
            row = lg[len(p) - 1 + t]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > tol * float(row.abs().max()):
                assert int(row.argmax()) == o[t], (len(p), t)
                checked += 1
    assert checked >= 40
    assert eng.sched.pool.num_free == eng.sched.pool.num_total
