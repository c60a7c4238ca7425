"""Host-side parts of Resevik in the layer-list family: config.json reader (layer runs of a repeated span), weight
fusion, the library subset a process serving such a model builds, the memory estimate, replay bookkeeping with
state slots, and self-consistency of the oracle."""
import json

import pytest
import torch

from gpustack_b200.config import LayerListConfig, ModelConfig
from gpustack_b200.scheduler import Request, SamplingParams, Scheduler
from gpustack_b200.weights import (layer_list_tensor_shapes, load_layer_list, load_layer_list_dir, random_layer_list_state,
                                   save_layer_list_checkpoint)
from oracle import resevik_oracle as O

F64 = torch.float64


def _cfg():
    att = {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 10, "scale": 0.4, "mask": {"size": 7}, "rot": {"base": 50.0, "dims": 6}}
    ret = {"heads": 2, "dim": 12, "vdim": 6, "decay": [0.97, 0.8], "rot": {"base": 300.0, "dims": 8}}
    lig = {"heads": 3, "dim": 10, "vdim": 14, "decay": [0.5, 0.93, 0.999]}
    moe = {"kind": "moe", "expert": {"ff": 18}, "router": {"experts": 5, "top": 2}}
    return {"architecture": "Resevik", "vocab": 131, "width": 52, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [{"type": "lightning", "mixer": lig, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": None},
                       {"type": "retention", "mixer": ret, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": moe}]}


def test_config_reader_round_trip_runs_and_rejections(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    assert c.to_dict() == d and LayerListConfig.from_dict(c.to_dict()) == c
    assert c.residual == "parallel" and c.norm == "rms" and c.has_state and c.embed_scale == 2.5
    # layers 1..2 three times, the embedding before passes two and three, each run with a cache / state of its own
    assert c.runs() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert c.runs() == [(l, again) for l, again in O.layer_runs(d)]
    lig, att, ret = c.layers[0].mixer, c.layers[1].mixer, c.layers[2].mixer
    assert (lig.kind, lig.feature, lig.rot, lig.k_scale, lig.out_norm, lig.gate_act) == ("linear_attention", "silu", None, 1.0, "all_heads", "sigmoid")
    assert (ret.feature, ret.rot.layout, ret.rot.dims, ret.out_norm, ret.gate_act) == (None, "half", 8, "per_head", "silu")
    assert abs(ret.k_scale - 12 ** -0.5) < 1e-12 and ret.decay == (0.97, 0.8)
    assert (att.window, att.values_are_keys, att.qk_unit_norm, att.rot.layout, att.sink, att.gate, att.qkv_bias) == \
        (7, True, True, "interleaved", False, False, False)
    assert not att.tile_sized                                            # 10-wide heads: the generic kernels
    e = c.layers[0].mlp.moe
    assert (e.experts, e.top, e.ff, e.score, e.renormalize, e.weight_on, e.act, e.identity) == (5, 2, 18, "sigmoid", False, "input", "silu", 0)
    # four attention runs (layer 1 three times, layer 3 once) hold keys and values; three runs of each recurrent layer hold state
    assert c.kv_bytes_per_token() == 4 * 2 * (10 + 10) * 2
    assert c.state_bytes_per_seq() == 4 * (3 * 10 * 14 + 3 * 2 * 12 * 6)
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert isinstance(ModelConfig.from_pretrained(str(tmp_path)), LayerListConfig)
    p = json.loads(json.dumps(d))
    del p["loop"], p["embedding"]
    cp = LayerListConfig.from_dict(p)
    assert cp.runs() == [(l, False) for l in range(4)] and cp.embed_scale == 1.0
    p["loop"] = {"start": 0, "stop": 4, "times": 2}
    assert [r for r in LayerListConfig.from_dict(p).runs() if r[1]] == [(0, True)]
    bad = [("type", "conv"), ("mlp", {"kind": "dense", "ff": 8})]
    for where, val in bad:
        x = json.loads(json.dumps(d))
        x["layers"][2][where] = val
        with pytest.raises(ValueError):
            LayerListConfig.from_dict(x)
    for path, val in ((("layers", 1, "mixer", "rot", "dims"), 12), (("layers", 1, "mixer", "vdim"), 8), (("layers", 1, "mixer", "kv_heads"), 3),
                      (("layers", 1, "mixer", "mask", "size"), 0), (("layers", 2, "mixer", "decay"), [0.5]),
                      (("layers", 0, "mlp", "router", "top"), 6), (("loop", "stop"), 5), (("loop", "times"), 0)):
        x = json.loads(json.dumps(d))
        t = x
        for k in path[:-1]:
            t = t[k]
        t[path[-1]] = val
        with pytest.raises(ValueError):
            LayerListConfig.from_dict(x)


def test_weight_fusion_layout_and_checkpoint_round_trip(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    assert {k: tuple(v) for k, v in layer_list_tensor_shapes(c).items()} == O.tensor_shapes(d)
    W = O.random_weights(d, seed=1)
    w = load_layer_list(c, lambda k: W[k], "cpu")
    l0, l1, l2 = w.layers[0], w.layers[1], w.layers[2]
    assert torch.equal(l0.proj, torch.cat([W["l0.mix." + n] for n in "qkvg"])) and torch.equal(l0.out_norm, W["l0.mix.norm"])
    assert torch.equal(l1.proj, torch.cat([W["l1.mix.q"], W["l1.mix.k"]])) and l1.norm2 is None and l1.router is None
    assert l2.out_norm is None and l2.decay.tolist() == pytest.approx([0.97, 0.8])
    assert l0.rot_freq is None and l1.rot_freq.dtype == torch.float64
    assert l1.rot_freq.tolist() == pytest.approx([50.0 ** (-2 * i / 6) for i in range(3)])
    assert l2.rot_freq.tolist() == pytest.approx([300.0 ** (-2 * i / 8) for i in range(4)])
    assert l0.router.shape == (128, 52) and torch.equal(l0.router[:5], W["l0.mlp.router"]) and not l0.router[5:].any()
    assert l0.correction is None and l0.w13.shape == (5 * 36, 52) and l0.w2.shape == (5 * 52, 18)
    assert torch.equal(l0.w13[36 * 3:36 * 4:2], W["l0.mlp.e3.gate"]) and torch.equal(l0.w13[36 * 3 + 1:36 * 4:2], W["l0.mlp.e3.up"])
    bad = dict(W)
    bad["l1.mix.k"] = W["l1.mix.k"][:-1]
    with pytest.raises(ValueError):
        load_layer_list(c, lambda k: bad[k], "cpu")
    st = random_layer_list_state(c, seed=2)
    assert set(st) == set(W)
    save_layer_list_checkpoint(c, st, str(tmp_path))
    back = load_layer_list_dir(ModelConfig.from_pretrained(str(tmp_path)), str(tmp_path), "cpu")
    assert torch.equal(back.layers[3].proj, torch.cat([st["l3.mix.q"], st["l3.mix.k"]]))


def test_library_subset_of_a_parallel_residual_model():
    import ctypes

    from gpustack_b200 import build

    c = LayerListConfig.from_dict(_cfg())
    tag, srcs = build.layer_list_sources(c)
    assert tag == "parallel_routed" and {"prenorm.cu", "rot_prep.cu", "linear_attn.cu", "attention_sink.cu", "moe_biased.cu", "moe.cu",
                                         "gemm_simt_grouped.cu"} <= set(srcs)
    assert "mlstm.cu" not in srcs and "latent.cu" not in srcs and "allreduce.cu" not in srcs and "attention_prefill_tc.cu" not in srcs
    d = _cfg()
    for l in d["layers"]:
        l["mlp"] = None
    assert build.layer_list_sources(LayerListConfig.from_dict(d))[0] == "parallel"
    h = ctypes.CDLL(str(build.build(sources=srcs, tag=tag)))
    for n in ("b200_add_rms_norm_f32", "b200_rot_prep", "b200_linattn_scan", "b200_linattn_out", "b200_attn_sink_prefill_ex",
              "b200_attn_sink_decode_ex", "b200_moe_route_scored", "b200_linear_simt_grouped_ex", "b200_moe_gather_scaled",
              "b200_moe_align", "b200_moe_combine_mixed", "b200_embed_streams", "b200_linear_simt", "b200_gemm_bf16_ex",
              "b200_moe_grouped_gemm_ex", "b200_sample_f32", "b200_last_error"):
        assert hasattr(h, n), n
    assert not hasattr(h, "b200_mlstm_scan") and not hasattr(h, "b200_latent_prep")


def test_vram_estimate_counts_every_run_of_a_repeated_layer():
    from gpustack_b200.config import EngineConfig
    from gpustack_b200.resource_fit import estimate

    d = _cfg()
    c = LayerListConfig.from_dict(d)
    e16 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256))
    e32 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256, dtype="float32"))
    assert e16.weights == c.weight_bytes() and e16.kv_bytes_per_token == c.kv_bytes_per_token()
    assert e32.kv_bytes_per_token == 2 * e16.kv_bytes_per_token and e32.workspace > e16.workspace
    n = sum(v.numel() for k, v in O.random_weights(d, 0).items() if "norm" not in k and k != "embed")
    assert c.weight_bytes() == 2 * n
    d["loop"]["times"] = 1
    once = LayerListConfig.from_dict(d)
    assert once.kv_bytes_per_token() == c.kv_bytes_per_token() // 2 and once.state_bytes_per_seq() < c.state_bytes_per_seq()
    assert once.weight_bytes() == c.weight_bytes()                       # the weights are shared by the passes


def test_replay_bookkeeping_with_state_slots():
    s = Scheduler(9, 16, 2, 256, 256, None, False, state_slots=2)
    a, b, c = (Request(req_id=i, prompt_ids=[], params=SamplingParams(max_tokens=0)) for i in "abc")
    s.replay_admit(a)
    s.replay_admit(b)
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(Exception):
        s.replay_admit(c)                                                # no third slot
    s.replay_extend(a, 40)
    freed = a.state_slot
    s.replay_finish(a)
    s.replay_admit(c)
    assert c.state_slot == freed and a.state_slot == -1                  # the freed slot goes to the next request
    s.replay_finish(b)
    s.replay_finish(c)
    assert s.pool.num_free == s.pool.num_total and s.slots.num_free == 2


def test_oracle_mechanisms_are_consistent():
    g = torch.Generator().manual_seed(0)
    T, H, dk, dv = 30, 2, 6, 5
    q, k = torch.randn(T, H, dk, generator=g, dtype=F64), torch.randn(T, H, dk, generator=g, dtype=F64)
    v = torch.randn(T, H, dv, generator=g, dtype=F64)
    decay = torch.tensor([0.9, 0.5], dtype=F64)
    # the recurrence equals the explicit sum  o_t = sum_{s<=t} d^(t-s) (q_t . k_s) v_s, and can be cut anywhere
    o, S = O.decayed_linear_attention(q, k, v, decay)
    t = 17
    want = sum(decay.reshape(H, 1) ** (t - s) * (q[t] * k[s]).sum(-1, keepdim=True) * v[s] for s in range(t + 1))
    assert torch.allclose(o[t], want, atol=1e-12)
    o1, S1 = O.decayed_linear_attention(q[:11], k[:11], v[:11], decay)
    o2, S2 = O.decayed_linear_attention(q[11:], k[11:], v[11:], decay, S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # a window as long as the sequence is plain causal attention; a window of one returns the position's own value
    kk, vv = k[:, :1], torch.randn(T, 1, dk, generator=g, dtype=F64)
    full = O.window_softmax_attention(q, kk, vv, 0.3, T)
    wide = O.window_softmax_attention(q, kk, vv, 0.3, 10 * T)
    assert torch.allclose(full, wide)
    one = O.window_softmax_attention(q, kk, vv, 0.3, 1)
    assert torch.allclose(one, vv.expand(T, H, dk))
    # rotation: scores depend on the distance only, both layouts; entries past `dims` pass
    pos = torch.arange(T)
    for layout in ("interleaved", "half"):
        a, b = O.rotate(q, pos, 100.0, 4, layout), O.rotate(k, pos, 100.0, 4, layout)
        a2, b2 = O.rotate(q, pos + 1000, 100.0, 4, layout), O.rotate(k, pos + 1000, 100.0, 4, layout)
        assert torch.allclose((a[9] * b[4]).sum(-1), (a2[9] * b2[4]).sum(-1), atol=1e-9)
        assert torch.equal(a[..., 4:], q[..., 4:]) and torch.equal(a[0], q[0])
    # the routing weight on the input is not the weight on the output (the expert is not linear)
    d = _cfg()
    W = {kk_: vv_.to(F64) for kk_, vv_ in O.sub(O.random_weights(d, 3), "l0.mlp.").items()}
    h = torch.randn(4, 52, generator=g, dtype=F64)
    ids, w = O.route_sigmoid(h, W["router"], 2)
    assert bool((w > 0).all()) and bool((w < 1).all()) and bool((w[:, 0] >= w[:, 1]).all())
    y = O.moe_ff(h, W, d["layers"][0]["mlp"])
    outside = sum(w[0, j] * O.expert(h[0], *(W[f"e{int(ids[0, j])}.{n}"] for n in ("gate", "up", "down"))) for j in range(2))
    assert not torch.allclose(y[0], outside, rtol=1e-3)
