"""Resevik (layer-list decoder: one norm per layer feeding mixer and feed-forward side by side, decayed linear
attention, rotary sliding-window attention whose values are its keys, sigmoid-routed experts weighted on their
input, a repeated span of layers) on the GPU against the plain restatement in oracle/resevik_oracle.py.

Every test builds its own small configuration and random weights.  Kernel tests compare one mechanism with the
oracle's function; engine tests drive LLMEngine (scheduler pools, state slots, runner step functions, CUDA graphs)
and compare logits with the oracle's whole-sequence forward.  float32 must agree to rounding, bfloat16 to bf16
rounding."""
import numpy as np
import pytest
import torch

from oracle import resevik_oracle as O

pytestmark = pytest.mark.gpu

F64 = torch.float64
BF = torch.bfloat16


def _attn(heads, kv_heads, dim, window, dims=None, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                                           "scale": scale or dim ** -0.5, "mask": {"size": window},
                                           "rot": {"base": base, "dims": dims or dim}}}


def _lin(kind, heads, dim, vdim, decay, dims=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if kind == "retention":
        m["rot"] = {"base": base, "dims": dims or dim}
    return {"type": kind, "mixer": m}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def cfg_odd():
    """Nothing is a multiple of 8: every product takes the CUDA-core path.  A lightning layer first; key and value
    widths that differ; rotations over part of the head; two of five experts; a layer without feed-forward; windows
    of 7 and 1; one key head for all query heads and one per query head; the middle layer alone runs three times."""
    return {"architecture": "Resevik", "vocab": 131, "width": 52, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
            "loop": {"start": 2, "stop": 3, "times": 3},
            "layers": [dict(_lin("lightning", 3, 10, 14, [0.5, 0.93, 0.9985]), mlp=_moe(5, 2, 18)),
                       dict(_attn(3, 1, 10, 7, dims=6, base=50.0, scale=0.4), mlp=None),
                       dict(_lin("retention", 2, 12, 6, [0.97, 0.8], dims=8, base=300.0), mlp=_moe(3, 3, 30)),
                       dict(_attn(2, 2, 14, 1, dims=14), mlp=_moe(4, 1, 22)),
                       dict(_attn(4, 2, 6, 40, dims=2, base=1e6, scale=1.5), mlp=_moe(2, 1, 10))]}


def cfg_tiles():
    """Widths that the tensor-core GEMMs take in bf16 (projections, grouped expert products with 256-wide rows and
    128-wide experts), 64-wide heads, a window of 24 that prompts and decoding pass, two layers that run twice."""
    return {"architecture": "Resevik", "vocab": 256, "width": 256, "embedding": {"scale": 16.0}, "norm": {"eps": 1e-6},
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [dict(_lin("retention", 2, 64, 128, [0.9, 0.995], dims=32, base=2e5), mlp=_moe(4, 2, 128)),
                       dict(_attn(4, 2, 64, 24, dims=16, base=3e5, scale=0.11), mlp=_moe(6, 1, 128)),
                       dict(_lin("lightning", 2, 32, 64, [0.6, 0.995]), mlp=_moe(2, 2, 256))]}


def cfg_plain():
    """Values a model may happen to make trivial: no repeated span, one expert of which one is chosen, one head, a
    window longer than every sequence, embedding scale 1, a decay of exactly 1, a full rotation."""
    return {"architecture": "Resevik", "vocab": 77, "width": 40, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "loop": {"start": 1, "stop": 1, "times": 1},
            "layers": [dict(_attn(1, 1, 8, 4096), mlp=_moe(1, 1, 16)),
                       dict(_lin("retention", 1, 8, 8, [1.0]), mlp=None),
                       dict(_lin("lightning", 2, 16, 4, [0.9, 0.25]), mlp=_moe(2, 2, 24))]}


CFGS = {"odd": cfg_odd, "tiles": cfg_tiles, "plain": cfg_plain}


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


def _close(got, want, dtype):
    """float32: every logit to rounding.  bfloat16: rounding may overturn a router's close call, which moves that
    position's logits by more than rounding does; so at most one position in twenty may be off (a fault of the
    cache, the state or the batch moves most of them), and the typical position must be well inside the tolerance."""
    if dtype == "float32":
        return _rel(got, want) < TOL[dtype]
    want = want.to(torch.float64).numpy() if isinstance(want, torch.Tensor) else np.asarray(want, dtype=np.float64)
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1) / np.abs(want).max()
    return float(np.mean(err > TOL[dtype])) <= 0.05 and float(np.median(err)) < TOL[dtype] / 2


def _rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------------------------ mechanisms, one at a time
@pytest.mark.parametrize("D", [37, 64, 200])
@pytest.mark.parametrize("xdt", [torch.float32, BF])
def test_residual_sum_of_up_to_three_addends_and_rms_norm(D, xdt):
    from gpustack_b200 import ops

    T, eps = 9, 1e-5
    x, a, b, c = (_rnd(T, D, seed=i, scale=1.0 + i) for i in range(4))
    w = (1.0 + 0.3 * _rnd(D, seed=9)).to(BF)
    for use in ((), ("a",), ("a", "b"), ("a", "b", "c"), ("c",)):
        z = x.to(F64)
        kw = {}
        for n, t in (("a", a), ("b", b), ("c", c)):
            if n in use:
                z = z + t.to(F64)
                kw[n] = t.cuda()
        xo, xb = torch.full((T, D), 7.0, device="cuda"), torch.zeros(T, D, dtype=xdt, device="cuda")
        ops.add_rms_norm(x.cuda(), w.cuda(), eps, x_out=xo, xb_out=xb, **kw)
        assert _rel(xo, z) < 1e-6
        assert _rel(xb, O.rms_norm(z, w.to(F64), eps)) < KTOL[xdt]
    # in place, the sum alone; then the gather form of the final norm
    xs = x.cuda().clone()
    ops.add_rms_norm(xs, None, eps, a=a.cuda(), x_out=xs)
    assert _rel(xs, x.to(F64) + a.to(F64)) < 1e-6
    rows = torch.tensor([5, 0, 8, 5], dtype=torch.int32)
    xb = torch.zeros(4, D, dtype=xdt, device="cuda")
    ops.add_rms_norm(x.cuda(), w.cuda(), eps, a=a.cuda(), b=b.cuda(), rows=rows.cuda(), xb_out=xb)
    z = (x.to(F64) + a.to(F64) + b.to(F64))[rows.long()]
    assert _rel(xb, O.rms_norm(z, w.to(F64), eps)) < KTOL[xdt]


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("H,G,dk,dims,pad", [(4, 2, 10, 6, 3), (8, 4, 64, 16, 3), (8, 4, 64, 16, 16), (2, 2, 128, 128, 0),
                                                 (3, 1, 7, 2, 0), (16, 2, 128, 64, 0), (5, 5, 32, 16, 8)])
def test_rotation_unit_norm_and_cache_rows_of_an_attention_whose_values_are_its_keys(dtype, H, G, dk, dims, pad):
    """Interleaved pairs, positions far from 0 (the angle must not lose digits), shuffled cache slots, a padding row:
    q in place, rotated and normed keys in the K pages, the keys as projected in the V pages.  Rows whose pitch is a
    multiple of 16 bytes take the 16-byte kernel, the others the element-wise one."""
    from gpustack_b200 import ops

    T, page, blocks, eps, base = 11, 16, 5, 1e-5, 3e5
    proj = _rnd(T, (H + G) * dk + pad, seed=1, dtype=dtype)
    pos = torch.tensor([0, 1, 2, 39, 40, 1000, 4095, 65537, 200001, 7, 8], dtype=torch.int32)
    slots = torch.randperm(blocks * page, generator=torch.Generator().manual_seed(2))[:T].to(torch.int32)
    slots[4] = -1
    kc = torch.full((blocks, G, page, dk), 9.0, dtype=dtype, device="cuda")
    vc = torch.full((blocks, G, page, dk), 9.0, dtype=dtype, device="cuda")
    i = torch.arange(dims // 2, dtype=F64)
    freq = (base ** (-2.0 * i / dims)).cuda()
    pd = proj.cuda().clone()
    ops.rot_prep(pd, 0, H * dk, -1, pos.cuda(), slots.cuda(), pd, kc, vc, H, G, dk, dk, paged=True, rot_dims=dims,
                 half_layout=False, freq=freq, unit_norm=True, eps=eps)
    q = proj[:, :H * dk].to(F64).reshape(T, H, dk)
    k = proj[:, H * dk:(H + G) * dk].to(F64).reshape(T, G, dk)
    qw = O.rms_norm(O.rotate(q, pos, base, dims, "interleaved"), None, eps)
    kw = O.rms_norm(O.rotate(k, pos, base, dims, "interleaved"), None, eps)
    assert _rel(pd[:, :H * dk], qw.reshape(T, -1)) < KTOL[dtype]
    assert torch.equal(pd[:, H * dk:].cpu(), proj[:, H * dk:])          # the key columns themselves stay as projected
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        assert _rel(kc[s // page, :, s % page], kw[t]) < KTOL[dtype]
        assert torch.equal(vc[s // page, :, s % page].cpu().to(F64), k[t])
    used = {int(s) for s in slots if s >= 0}
    free = [s for s in range(blocks * page) if s not in used]
    assert all(float(kc[s // page, 0, s % page, 0]) == 9.0 for s in free)


@pytest.mark.parametrize("src", [torch.float32, BF])
@pytest.mark.parametrize("feature,dims,half", [("silu", 0, False), (None, 12, True), (None, 8, True), ("silu", 4, False),
                                               (None, 32, True), (None, 16, True), ("silu", 16, False)])
@pytest.mark.parametrize("H,dk,dv", [(3, 12, 10), (3, 32, 16), (8, 128, 128)])
def test_feature_map_rotation_and_key_factor_into_fp32_rows(src, feature, dims, half, H, dk, dv):
    from gpustack_b200 import ops

    if dims > dk:
        pytest.skip("rotation wider than the head")
    T, base = 7, 300.0
    kc, vc = H * dk, 2 * H * dk
    proj = _rnd(T, vc + 2 * H * dv, seed=3, dtype=src)
    pos = torch.tensor([0, 1, 5, 77, 1023, 30000, 123457], dtype=torch.int32)
    x32 = torch.zeros(T, vc + H * dv, device="cuda")
    freq = None
    if dims:
        freq = (base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)).cuda()
    ops.rot_prep(proj.cuda(), 0, kc, vc, pos.cuda(), None, x32, x32[:, kc:], x32[:, vc:], H, H, dk, dv, paged=False,
                 feature=feature, rot_dims=dims, half_layout=half, freq=freq, k_mul=dk ** -0.5)
    f = O.silu if feature else (lambda z: z)
    q = f(proj[:, :kc].to(F64)).reshape(T, H, dk)
    k = f(proj[:, kc:vc].to(F64)).reshape(T, H, dk)
    v = f(proj[:, vc:vc + H * dv].to(F64))
    if dims:
        q = O.rotate(q, pos, base, dims, "half" if half else "interleaved")
        k = O.rotate(k, pos, base, dims, "half" if half else "interleaved")
    tol = 2e-6 if src == torch.float32 else 2e-6      # the source is exact in fp64 either way; the result is fp32
    assert _rel(x32[:, :kc], q.reshape(T, -1)) < tol
    assert _rel(x32[:, kc:vc], k.reshape(T, -1) * dk ** -0.5) < tol
    assert _rel(x32[:, vc:], v) < tol


def _scan(x32, H, dk, dv, decay, lens_per_step, S, slot=0, other=None):
    """Run one sequence through the kernel in portions; `other` = (rows, state slot) of a second sequence whose single
    rows ride in the same launches."""
    from gpustack_b200 import ops

    kc, vc = H * dk, 2 * H * dk
    outs, at, oat = [], 0, 0
    for n in lens_per_step:
        rows = [x32[at:at + n]]
        cu, ctx, sl = [0, n], [at], [slot]
        if other is not None and oat < other[0].shape[0]:
            rows.append(other[0][oat:oat + 1])
            cu.append(n + 1)
            ctx.append(oat)
            sl.append(other[1])
            oat += 1
        xin = torch.cat(rows).cuda()
        o = torch.zeros(xin.shape[0], H * dv, device="cuda")
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")   # noqa: E731
        ops.linattn_scan(xin, 0, kc, vc, decay.cuda(), i32(cu), i32(ctx), i32(sl), S, o, H, dk, dv, max_len=n)
        outs.append(o[:n].cpu())
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("H,dk,dv", [(3, 10, 14), (2, 64, 64), (1, 128, 40), (2, 33, 70)])
@pytest.mark.parametrize("cut", ["whole", "single", "mixed"])
def test_decayed_linear_attention_in_portions_against_the_recurrence(H, dk, dv, cut):
    """Chunk form, serial form and any mixture give the recurrence's outputs and final state; a slot that held another
    sequence (here: NaN) starts from zero; a second sequence's single rows in the same launches do not disturb it."""
    n = 83
    x32 = _rnd(n, 2 * H * dk + H * dv, seed=4, scale=0.5)
    decay = torch.tensor([0.55, 0.97, 0.9995][:H] if H <= 3 else [0.9] * H)
    q = x32[:, :H * dk].to(F64).reshape(n, H, dk)
    k = x32[:, H * dk:2 * H * dk].to(F64).reshape(n, H, dk)
    v = x32[:, 2 * H * dk:].to(F64).reshape(n, H, dv)
    want, Sw = O.decayed_linear_attention(q, k, v, decay.to(F64))
    lens = {"whole": [n], "single": [1] * n, "mixed": [2, 3, 16, 17, 1, 1, 2, 31, 5, 2, 3]}[cut]
    assert sum(lens) == n
    S = torch.full((3, H, dv, dk), float("nan"), device="cuda")
    x2 = _rnd(40, 2 * H * dk + H * dv, seed=5, scale=0.5)
    got = _scan(x32, H, dk, dv, decay, lens, S, slot=1, other=(x2, 2) if cut != "whole" else None)
    assert _rel(got, want.reshape(n, -1)) < 2e-5
    assert _rel(S[1], Sw.transpose(1, 2)) < 2e-5
    assert bool(torch.isnan(S[0]).all())
    if cut != "whole":
        m = min(len(lens), 40)
        S2 = O.decayed_linear_attention(x2[:m, :H * dk].to(F64).reshape(m, H, dk), x2[:m, H * dk:2 * H * dk].to(F64).reshape(m, H, dk),
                                        x2[:m, 2 * H * dk:].to(F64).reshape(m, H, dv), decay.to(F64))[1]
        assert _rel(S[2], S2.transpose(1, 2)) < 2e-5


def test_a_key_far_back_survives_a_slow_decay_and_dies_under_a_fast_one():
    """One key / value pair at position 3 made large; 400 positions later the slow head still returns it (times
    decay^397), the fast head has lost it: the state is carried across portions and single rows, not rebuilt."""
    H, dk, dv, n = 2, 16, 16, 404
    x32 = _rnd(n, 2 * H * dk + H * dv, seed=6, scale=0.05)
    kc, vc = H * dk, 2 * H * dk
    probe = torch.zeros(dk)
    probe[5] = 1.0
    for h in range(H):
        x32[3, kc + h * dk:kc + (h + 1) * dk] = 40.0 * probe
        x32[3, vc + h * dv:vc + (h + 1) * dv] = torch.arange(1, dv + 1, dtype=torch.float32)
        x32[n - 1, h * dk:(h + 1) * dk] = probe
    decay = torch.tensor([0.999, 0.5])
    q = x32[:, :kc].to(F64).reshape(n, H, dk)
    k = x32[:, kc:vc].to(F64).reshape(n, H, dk)
    v = x32[:, vc:].to(F64).reshape(n, H, dv)
    want, _ = O.decayed_linear_attention(q, k, v, decay.to(F64))
    S = torch.zeros(1, H, dv, dk, device="cuda")
    got = _scan(x32, H, dk, dv, decay, [100, 2, 150] + [1] * 152, S)
    assert _rel(got[-1], want[-1].reshape(-1)) < 2e-5
    slow, fast = got[-1, :dv], got[-1, dv:]
    assert float(slow[-1]) > 0.5 * 40.0 * dv * 0.999 ** 400 and float(fast.abs().max()) < 1.0


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("all_heads,gate", [(True, "sigmoid"), (False, "silu"), (False, "sigmoid")])
def test_output_norm_and_gate_of_the_linear_mixers(dtype, all_heads, gate):
    from gpustack_b200 import ops

    T, H, dv, eps = 6, 3, 14, 1e-5
    o = _rnd(T, H * dv, seed=7, scale=3.0)
    proj = _rnd(T, 5 + H * dv, seed=8, dtype=dtype)
    w = (1.0 + 0.3 * _rnd(H * dv, seed=9)).to(BF) if all_heads else None
    out = torch.zeros(T, H * dv, dtype=dtype, device="cuda")
    ops.linattn_out(o.cuda(), proj.cuda(), 5, None if w is None else w.cuda(), out, H, dv, eps, all_heads, gate)
    g = proj[:, 5:].to(F64)
    act = torch.sigmoid(g) if gate == "sigmoid" else O.silu(g)
    if all_heads:
        want = O.rms_norm(o.to(F64), w.to(F64), eps) * act
    else:
        want = O.rms_norm(o.to(F64).reshape(T, H, dv), None, eps).reshape(T, -1) * act
    assert _rel(out, want) < KTOL[dtype]


def _window_case(dtype, n, H, G, dk, window, seed, stand=None):
    """A sequence of n keys in shuffled pages (junk elsewhere); q rows for every position.  stand = (i, j): key j is
    made to dominate query i's scores if it is visible."""
    page = 16
    nb = (n + page - 1) // page
    q, k, v = _rnd(n, H, dk, seed=seed), _rnd(n, G, dk, seed=seed + 1), _rnd(n, G, dk, seed=seed + 2)
    if stand is not None:
        i, j = stand
        for g in range(G):
            k[j, g] = 6.0 * q[i, g * (H // G)] / q[i, g * (H // G)].norm() * dk ** 0.5
            v[j, g] = 10.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed))[:nb]
    kc = torch.full((nb + 3, G, page, dk), 50.0, dtype=dtype)
    vc = torch.full((nb + 3, G, page, dk), -50.0, dtype=dtype)
    for t in range(n):
        kc[perm[t // page], :, t % page] = k[t]
        vc[perm[t // page], :, t % page] = v[t]
    return q, k, v, kc.cuda(), vc.cuda(), perm.to(torch.int32)


def _run_window(q, kc, vc, perm, H, G, dk, window, scale, start, n):
    """Rows [start, n) as one prompt portion (context `start`), then the last row again through the decode kernel."""
    from gpustack_b200 import ops

    dtype = q.dtype
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")   # noqa: E731
    rows = q[start:n].reshape(n - start, H * dk).cuda().contiguous()
    out = torch.zeros_like(rows)
    ts, tq = ops.build_prefill_tiles([n - start], ops.attn_sink_prefill_tile(), [start])
    bt = perm.cuda().reshape(1, -1)
    ops.attn_sink_prefill(rows, -1, kc, vc, bt, i32([0, n - start]), i32([start]), i32(ts), i32(tq), None, out, H, G, dk, dk,
                          scale, window=window)
    last = q[n - 1:n].reshape(1, H * dk).cuda().contiguous()
    od = torch.zeros_like(last)
    ops.attn_sink_decode(last, -1, kc, vc, bt, i32([n]), None, od, H, G, dk, dk, scale, window=window)
    return out.cpu(), od.cpu(), dtype


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("H,G,dk,window,n,start", [(3, 1, 10, 7, 70, 0), (4, 2, 64, 48, 150, 33), (2, 2, 14, 1, 40, 5),
                                                   (8, 4, 64, 33, 100, 64), (2, 1, 8, 500, 90, 17)])
def test_sliding_window_attention_over_shuffled_pages(dtype, H, G, dk, window, n, start):
    scale = 0.3
    q, k, v, kc, vc, perm = _window_case(dtype, n, H, G, dk, window, seed=11)
    want = O.window_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, window).reshape(n, -1)
    out, od, _ = _run_window(q, kc, vc, perm, H, G, dk, window, scale, start, n)
    assert _rel(out, want[start:]) < KTOL[dtype]
    assert _rel(od, want[n - 1:]) < KTOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("window,i", [(7, 60), (16, 47), (17, 48), (32, 95), (33, 64), (40, 100), (1, 20), (64, 127)])
@pytest.mark.parametrize("inside", [True, False])
def test_a_key_just_inside_the_window_dominates_and_just_outside_is_unseen(dtype, window, i, inside):
    """Key j = i - window + 1 is the last one query i sees, j = i - window the first it does not: made large, the first
    takes the whole softmax (the output is its value, 10), the second changes nothing.  Checked for a prompt row (with
    portions that start before, at and after the key) and for the decode kernel; edges at page and key-block borders."""
    H, G, dk, scale = 2, 1, 16, 1.0
    j = i - window + 1 if inside else i - window
    n = i + 1
    q, k, v, kc, vc, perm = _window_case(dtype, n, H, G, dk, window, seed=13, stand=(i, j))
    want = O.window_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, window).reshape(n, -1)
    assert (float(want[i, :dk].min()) > 9.9) == inside          # head 0 is the one the key was aligned with
    for start in sorted({0, max(0, j - 3), j, min(i, j + 1), i}):
        out, od, _ = _run_window(q, kc, vc, perm, H, G, dk, window, scale, start, n)
        assert _rel(out, want[start:]) < KTOL[dtype], start
        assert _rel(od, want[i:]) < KTOL[dtype]


def _run_window_tc(q, kc, vc, perm, H, G, dk, window, scale, start, n, splits):
    """The tensor-core routes (tcgen05 prefill tiles, split-KV decode) over the same cache."""
    from gpustack_b200 import ops

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")   # noqa: E731
    rows = q[start:n].reshape(n - start, H * dk).cuda().contiguous()
    out = torch.zeros_like(rows)
    ts, tq = ops.build_prefill_tiles([n - start], ops.attn_prefill_tile(H, G), [start])
    bt = perm.cuda().reshape(1, -1)
    ops.paged_attn_prefill_ex(rows, rows.stride(0), kc, vc, bt, i32([0, n - start]), i32([start]), i32(ts), i32(tq), out, H, G,
                              dk, scale, window=window)
    last = q[n - 1:n].reshape(1, H * dk).cuda().contiguous()
    od = torch.zeros_like(last)
    ws = ops.attn_decode_workspace(1, H, dk, splits, "cuda")
    ops.paged_attn_decode(last, last.stride(0), kc, vc, bt, i32([n]), od, H, G, dk, scale, num_splits=splits, workspace=ws,
                          window=window)
    return out.cpu(), od.cpu()


@pytest.mark.parametrize("window,n,start,splits", [(40, 300, 0, 1), (64, 300, 33, 3), (65, 257, 64, 2), (200, 300, 100, 4),
                                                   (1, 130, 7, 1), (1000, 300, 0, 2), (129, 400, 250, 8)])
@pytest.mark.parametrize("H,G", [(8, 2), (8, 1)])
def test_sliding_window_on_the_tensor_core_attention_kernels(window, n, start, splits, H, G):
    """128-wide heads in groups of four and eight, bf16: the tcgen05 prefill kernel skips the key blocks before a tile's
    window and masks inside the first one; the split-KV decode kernel divides only the window's pages among its splits."""
    dk, scale = 128, 0.09
    q, k, v, kc, vc, perm = _window_case(BF, n, H, G, dk, window, seed=17)
    want = O.window_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, window).reshape(n, -1)
    out, od = _run_window_tc(q, kc, vc, perm, H, G, dk, window, scale, start, n, splits)
    assert _rel(out, want[start:]) < KTOL[BF]
    assert _rel(od, want[n - 1:]) < KTOL[BF]


@pytest.mark.parametrize("window,i", [(64, 127), (65, 128), (33, 200), (128, 191), (40, 100), (1, 70)])
@pytest.mark.parametrize("inside", [True, False])
def test_window_edges_on_the_tensor_core_attention_kernels(window, i, inside):
    H, G, dk, scale = 8, 2, 128, 0.25
    j = i - window + 1 if inside else i - window
    n = i + 1
    q, k, v, kc, vc, perm = _window_case(BF, n, H, G, dk, window, seed=19, stand=(i, j))
    want = O.window_softmax_attention(q.to(F64), k.to(F64), v.to(F64), scale, window).reshape(n, -1)
    assert (float(want[i, :dk].min()) > 9.9) == inside
    for start in sorted({0, max(0, j - 3), j, i}):
        out, od = _run_window_tc(q, kc, vc, perm, H, G, dk, window, scale, start, n, 2)
        assert _rel(out, want[start:]) < KTOL[BF], start
        assert _rel(od, want[i:]) < KTOL[BF]


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("D,E,top,ff", [(52, 5, 2, 18), (40, 1, 1, 16), (24, 3, 3, 30), (256, 4, 2, 128), (256, 70, 4, 128)])
def test_sigmoid_routed_experts_weighted_on_their_input(dtype, D, E, top, ff):
    """Scores are sigmoids, the `top` largest are chosen and are the weights as they are, each chosen expert runs on
    weight * x.  bf16 with 256-wide rows and 128-wide experts takes the grouped tensor-core products."""
    from gpustack_b200 import ops
    from gpustack_b200.weights import _interleave_rows

    T = 37
    x = _rnd(T, D, seed=21).to(dtype)
    W = {"router": (2.0 * _rnd(E, D, seed=22) / D ** 0.5).to(BF)}
    for e in range(E):
        W[f"e{e}.gate"] = (_rnd(ff, D, seed=30 + 3 * e) / D ** 0.5).to(BF)
        W[f"e{e}.up"] = (_rnd(ff, D, seed=31 + 3 * e) / D ** 0.5).to(BF)
        W[f"e{e}.down"] = (_rnd(D, ff, seed=32 + 3 * e) / ff ** 0.5).to(BF)
    want = O.moe_ff(x.to(F64), {k: v.to(F64) for k, v in W.items()}, {"router": {"experts": E, "top": top}})
    router = torch.zeros(-(-E // 128) * 128, D, dtype=BF)
    router[:E] = W["router"]
    w13 = torch.cat([_interleave_rows(W[f"e{e}.gate"], W[f"e{e}.up"]) for e in range(E)]).cuda()
    w2 = torch.cat([W[f"e{e}.down"] for e in range(E)]).cuda()
    ws = ops.RoutedWorkspace(T, top, E, D, ff, dtype, "cuda")
    out = torch.zeros(T, D, device="cuda")
    ops.routed_experts(x.cuda(), router.cuda(), None, w13, w2, ws, out, E, 0, top, 1.0, ff, 0.0, sigmoid=True,
                       renormalize=False, weight_on="input", act="silu")
    ids, wt = O.route_sigmoid(x.to(F64), W["router"].to(F64), top)
    got_ids = ws.topk_ids[:T * top].view(T, top).cpu().long()
    if dtype == torch.float32:
        assert torch.equal(got_ids, ids)
        assert _rel(ws.topk_w[:T * top].view(T, top), wt) < 1e-5
        assert _rel(out, want) < 2e-5
    else:
        err = (out.cpu().to(F64) - want).abs().max(dim=1).values / want.abs().max()
        assert float((err > 3e-2).float().mean()) <= 0.06 and float(err.median()) < 1.5e-2


# ---------------------------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=list(CFGS))
def model(request):
    cfg = CFGS[request.param]()
    return cfg, O.random_weights(cfg, seed=3 + len(request.param))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer_run(model, dtype):
    cfg, W = model
    toks = _tokens(cfg, 70, 1)
    trail = []
    want = O.forward(cfg, W, toks, layer_outputs=trail)
    eng = _engine(cfg, W, dtype)
    seen = eng.runner.layer_trace = []
    got = eng.replay_step([("a", toks, list(range(len(toks))))], ["a"])
    eng.runner.layer_trace = None
    assert len(seen) == len(O.layer_runs(cfg)) == len(trail)
    for l in range(len(seen)):
        assert _rel(seen[l], trail[l]) < TOL[dtype] * 2, f"residual stream after layer run {l}"
    assert _close(got, want, dtype)
    # the serving path (sums folded into the next norm) gives the same logits as the traced one
    again = eng.replay_step([("b", toks, list(range(len(toks))))], ["b"])
    assert _rel(again, got) < (1e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_single_tokens_match_the_whole_prompt(model, dtype):
    """One prompt, token by token, and portions of changing size down to two tokens (page size 16, chunks of 16, windows
    of 1 / 7 / 24 / 40: cuts inside and at their borders): the logits at a position do not depend on the cut."""
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
    portions of some ride beside single tokens of others, a finished request's pages and state slot go to the next
    one (whose recurrence must start from zero).  Every request's logits equal those of the request alone."""
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
    """A random model: layer kinds, order, head counts, widths (odd and tile-sized), windows, decays, rotations,
    experts and the repeated span all drawn anew."""
    D = rng.choice([48, 64, 96, 128, 192, 256, 320])
    n = rng.randint(2, 6)
    layers = []
    for _ in range(n):
        kind = rng.choice(["attention", "retention", "lightning"])
        if kind == "attention":
            G = rng.choice([1, 2, 3, 4])
            dk = rng.choice([8, 16, 20, 24, 32, 64, 128])
            layer = _attn(G * rng.choice([1, 2, 3, 4, 5]), G, dk, rng.choice([1, 2, 5, 16, 17, 33, 48, 64, 100, 1000]),
                          dims=rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dk]), base=rng.choice([100.0, 1e4, 3e5]),
                          scale=rng.choice([dk ** -0.5, 0.2]))
        else:
            H, dk, dv = rng.choice([1, 2, 3, 4, 6]), rng.choice([8, 12, 16, 20, 32, 64, 128]), rng.choice([8, 12, 16, 32, 40, 64, 128])
            layer = _lin(kind, H, dk, dv, [rng.choice([0.3, 0.6, 0.9, 0.99, 0.9985, 1.0]) for _ in range(H)],
                         dims=rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dk]), base=rng.choice([100.0, 1e4, 1e6]))
        E = rng.choice([1, 2, 4, 8, 16])
        layers.append(dict(layer, mlp=_moe(E, rng.randint(1, min(E, 4)), rng.choice([16, 24, 64, 96, 128, 256])) if rng.random() < 0.8 else None))
    a = rng.randint(0, n)
    return {"architecture": "Resevik", "vocab": rng.choice([100, 257, 1000]), "width": D, "embedding": {"scale": rng.choice([1.0, D ** 0.5])},
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers,
            "loop": {"start": a, "stop": rng.randint(a, n), "times": rng.choice([1, 2, 3])}}


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106])
def test_random_configurations_in_float32(seed):
    """Whole prompt, and two requests in portions beside single tokens, against the oracle (fp32: no router call is
    close enough for rounding to overturn it)."""
    import random

    cfg = _random_cfg(random.Random(seed))
    W = O.random_weights(cfg, seed=seed)
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
    """300 single-token steps after a short prompt through the captured decode graphs: every window slides over
    decoded tokens many times, the decode kernel walks 20 pages, the recurrent states pass through 300 updates."""
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
