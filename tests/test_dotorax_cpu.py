"""Host-side parts of Dotorax in the layer-list family: config.json reader, weight fusion, the library subset a
process serving such a model builds, the memory estimate, and self-consistency of the oracle."""
import json

import pytest
import torch

from gpustack_b200.config import LayerListConfig, ModelConfig
from gpustack_b200.weights import (layer_list_tensor_shapes, load_layer_list, load_layer_list_dir, random_layer_list_state,
                                   save_layer_list_checkpoint)
from oracle import dotorax_oracle as O

F64 = torch.float64


def _cfg():
    att = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "rot": {"base": 300.0, "dims": 4}}
    left = {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 6, "scale": 0.9, "rot": {"base": 50.0, "dims": 6},
            "mask": {"size": 7, "pool": 3}}
    par = {"left": left, "right": {"width": 21, "blocks": 3, "conv": 2}, "left_scale": 0.4, "right_scale": 1.3}
    gla = {"heads": 3, "dim": 10, "vdim": 14, "tau": 3.0}
    ff = {"kind": "dense", "ff": 18, "limit": 1.5}
    return {"architecture": "Dotorax", "vocab": 131, "width": 52, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "canon": {"taps": 4}, "max_positions": 300,
            "layers": [{"type": "gla", "mixer": gla, "mlp": ff}, {"type": "parallel", "mixer": par, "mlp": None},
                       {"type": "attention", "mixer": att, "mlp": ff},
                       {"type": "attention", "mixer": dict(att, kv_from=2), "mlp": ff}]}


def test_config_reader_round_trip_and_rejections(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    assert c.family == "layer_list" and c.residual == "sandwich" and c.norm == "rms_zero_centred" and c.canon_taps == 4
    assert c.learned_positions and c.max_position_embeddings == 300 and c.residual_mult == 0.7 and c.has_state
    g, p, a, b = (l.mixer for l in c.layers)
    assert g.kind == "gated_linear_attention" and (g.heads, g.dim, g.vdim, g.tau) == (3, 10, 14, 3.0)
    assert p.kind == "side_by_side" and p.left.window == 7 and p.left.pool == 3 and p.left.qk_unit_norm and p.left.head_temp
    assert p.left.rot.layout == "interleaved" and not p.left.gate and (p.left_scale, p.right_scale) == (0.4, 1.3)
    assert (p.right.width, p.right.blocks, p.right.conv) == (21, 3, 2) and c.layers[1].mlp is None
    assert a.kind == "attention" and a.gate and a.gate_per_head and a.gate_width == 4 and a.rot.layout == "half" and not a.window
    assert b.kv_from == 2 and c.kv_owner(3) == 2 and c.kv_owner(1) == 1 and c.kv_owner(0) is None
    assert c.layers[0].mlp.act == "clamped_swish" and c.layers[0].mlp.limit == 1.5
    assert not a.tile_sized and not p.left.tile_sized      # 6-wide keys; pooled blocks are not on the tensor-core kernels
    assert p.left.pool_per_page(16) == 6
    back = LayerListConfig.from_dict(json.loads(json.dumps(c.to_dict())))
    assert back == c
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert ModelConfig.from_pretrained(str(tmp_path)) == c
    # a model without positions of its own in the request is still bounded by its table
    for breaker in (lambda x: x["layers"][3]["mixer"].update(kv_from=1),            # not an attention layer
                    lambda x: x["layers"][3]["mixer"].update(kv_from=3),            # not an earlier layer
                    lambda x: x["layers"][3]["mixer"].update(heads=8),              # head shapes differ from the owner's
                    lambda x: x["layers"][2]["mixer"]["rot"].update(dims=7),
                    lambda x: x["layers"][1]["mixer"]["left"]["mask"].update(pool=0),
                    lambda x: x["layers"][1]["mixer"]["right"].update(blocks=4),
                    lambda x: x["layers"][0]["mixer"].update(tau=0.0),
                    lambda x: x["layers"][0].update(type="mamba"),
                    lambda x: x["layers"][0]["mlp"].update(kind="moe")):
        bad = json.loads(json.dumps(d))
        breaker(bad)
        with pytest.raises((ValueError, KeyError)):
            LayerListConfig.from_dict(bad)
    one = json.loads(json.dumps(d))
    one["canon"]["taps"] = 1
    for l in one["layers"]:
        if l["type"] != "attention":
            l["type"], l["mixer"] = "attention", dict(one["layers"][2]["mixer"])
    one["layers"][3]["mixer"]["kv_from"] = 2
    assert not LayerListConfig.from_dict(one).has_state              # attention alone, one tap: nothing is carried


def test_weight_fusion_layout_and_checkpoint_round_trip(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    W = O.random_weights(d, seed=1, decay_rank=5)
    w = load_layer_list(c, lambda k: W[k], "cpu")
    assert c.layers[0].mixer.decay_rank == 5                           # taken from the checkpoint
    assert {k: tuple(v) for k, v in layer_list_tensor_shapes(c).items()} == O.tensor_shapes(d, 5)
    l0, l1, l2, l3 = w.layers
    rows = torch.cat([W["l0.mix." + n] for n in ("q", "k", "v", "g", "a1")])
    assert l0.proj.shape[0] % 8 == 0 and torch.equal(l0.proj[:rows.shape[0]], rows) and not l0.proj[rows.shape[0]:].any()
    assert torch.equal(l0.decay_up, W["l0.mix.a2"]) and torch.equal(l0.out_norm, W["l0.mix.norm"])
    assert l0.canon1.dtype == torch.float32 and torch.equal(l0.canon1, W["l0.canon1"].float()) and l0.canon2 is not None
    assert torch.equal(l0.norm1b, W["l0.norm1b"]) and torch.equal(l0.norm2b, W["l0.norm2b"])
    assert torch.equal(l0.gate_up[0::2], W["l0.mlp.gate"]) and torch.equal(l0.gate_up[1::2], W["l0.mlp.up"])
    rows = torch.cat([W["l1.mix.left.q"], W["l1.mix.left.k"], W["l1.mix.left.v"], W["l1.mix.right.y"], W["l1.mix.right.x"]])
    assert torch.equal(l1.proj[:rows.shape[0]], rows) and l1.norm2 is None and l1.canon2 is None and l1.gate_up is None
    assert torch.equal(l1.o, W["l1.mix.left.o"]) and torch.equal(l1.o2, W["l1.mix.right.o"])
    assert torch.equal(l1.head_scale, W["l1.mix.left.temp"].float())
    assert torch.equal(l1.rec_bias, torch.cat([W["l1.mix.right.y.b"], W["l1.mix.right.x.b"]]).float())
    assert torch.equal(l1.rec_gates, torch.cat([W["l1.mix.right.ra"], W["l1.mix.right.ri"]])) and l1.rec_gates.shape == (6, 7, 7)
    assert torch.equal(l1.rec_gate_bias, torch.cat([W["l1.mix.right.ra.b"].reshape(-1), W["l1.mix.right.ri.b"].reshape(-1)]).float())
    assert l1.rot_freq.tolist() == pytest.approx([50.0 ** (-2 * i / 6) for i in range(3)])
    rows = torch.cat([W["l2.mix." + n] for n in "qkvg"])
    assert torch.equal(l2.proj[:rows.shape[0]], rows)
    rows = torch.cat([W["l3.mix.q"], W["l3.mix.g"]])
    assert torch.equal(l3.proj[:rows.shape[0]], rows) and "l3.mix.k" not in W
    assert torch.equal(w.pos, W["pos"]) and w.pos.shape == (300, 52)
    bad = dict(W)
    bad["l1.mix.right.ra"] = W["l1.mix.right.ra"][:-1]
    with pytest.raises(ValueError):
        load_layer_list(c, lambda k: bad[k], "cpu")
    st = random_layer_list_state(c, seed=2)
    assert set(st) == set(W)
    save_layer_list_checkpoint(c, st, str(tmp_path))
    back = load_layer_list_dir(ModelConfig.from_pretrained(str(tmp_path)), str(tmp_path), "cpu")
    assert torch.equal(back.layers[3].proj[:28], torch.cat([st["l3.mix.q"], st["l3.mix.g"]]))


def test_library_subset_of_a_sandwich_residual_model():
    import ctypes

    from gpustack_b200 import build

    c = LayerListConfig.from_dict(_cfg())
    tag, srcs = build.layer_list_sources(c)
    assert tag == "sandwich" and {"sandwich.cu", "rot_prep.cu", "attention_sink.cu", "gated_recurrence.cu", "gated_linear_attn.cu",
                                  "linear_attn.cu", "gemm_simt_grouped.cu"} <= set(srcs)
    assert "mlstm.cu" not in srcs and "latent.cu" not in srcs and "allreduce.cu" not in srcs and "moe.cu" not in srcs
    h = ctypes.CDLL(str(build.build(sources=srcs, tag=tag)))
    for n in ("b200_embed_pos_f32", "b200_sandwich_join", "b200_causal_conv", "b200_conv_commit", "b200_kv_pool_update",
              "b200_attn_sink_prefill_pool", "b200_attn_sink_decode_pool", "b200_gated_recurrence_scan", "b200_gla_scan",
              "b200_rot_prep", "b200_linattn_out", "b200_linear_simt", "b200_linear_simt_grouped", "b200_gemm_bf16_ex",
              "b200_gemm_bf16_gated", "b200_sample_f32", "b200_last_error"):
        assert hasattr(h, n), n
    assert not hasattr(h, "b200_mlstm_scan") and not hasattr(h, "b200_latent_prep")
    # tile-sized heads in the windowed attention alone (pooled blocks follow): the tensor-core attention sources join,
    # since the window's tokens run on them
    d = _cfg()
    d["layers"][1]["mixer"]["left"].update(dim=64, vdim=64, rot={"base": 50.0, "dims": 16})
    w = LayerListConfig.from_dict(d)
    assert w.layers[1].mixer.left.tokens_tile_sized and not w.layers[1].mixer.left.tile_sized
    tag, srcs = build.layer_list_sources(w)
    assert tag == "sandwich_tc" and {"attention.cu", "attention_prefill_tc.cu"} <= set(srcs)


def test_vram_estimate_counts_pooled_blocks_rings_and_states():
    from gpustack_b200.config import EngineConfig
    from gpustack_b200.resource_fit import estimate

    d = _cfg()
    c = LayerListConfig.from_dict(d)
    e16 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256))
    e32 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256, dtype="float32"))
    assert e16.weights == c.weight_bytes() and e16.kv_bytes_per_token == c.kv_bytes_per_token()
    assert e32.kv_bytes_per_token > e16.kv_bytes_per_token and e32.workspace > e16.workspace
    # keys and values of the two owning layers in bf16, plus 6 fp32 block means per 16-token page of the pooled layer
    assert c.kv_bytes_per_token() == 2 * (2 * (6 + 10) + 1 * (10 + 6)) + 1 * (10 + 6) * 4 * 6 // 16
    # states: gla 3 x 10 x 14, recurrence 21 with one ring entry of 21, and 3 ring entries of 52 for the 7 sublayers
    assert c.state_bytes_per_seq() == 4 * (3 * 10 * 14 + 21 * 2 + 52 * 3 * 7)
    W = O.random_weights(d, 0, decay_rank=16)
    n = sum(v.numel() for k, v in W.items() if k.split(".")[-1] not in ("norm", "norm1", "norm2", "norm1b", "norm2b", "canon1",
            "canon2", "b", "temp", "lam", "conv", "pos", "embed"))
    assert c.weight_bytes() == 2 * n


def test_oracle_mechanisms_are_consistent():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)   # noqa: E731
    # the convolution against torch's, and its last tap on the current token
    x, w = r(20, 5), r(5, 3)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T.unsqueeze(0), (2, 0)), w.unsqueeze(1), groups=5)[0].T
    assert torch.allclose(O.causal_conv(x, w), ref)
    assert torch.allclose(O.causal_conv(x, w)[0], w[:, 2] * x[0])
    # a pool of one token makes every token before the window its own block: full causal attention
    q, k, v = r(40, 4, 6), r(40, 2, 6), r(40, 2, 5)
    full = O.causal_attention(q, k, v, 0.4)
    assert torch.allclose(O.pooled_window_attention(q, k, v, torch.full((4,), 0.4, dtype=F64), 7, 1), full)
    assert torch.allclose(O.pooled_window_attention(q, k, v, torch.full((4,), 0.4, dtype=F64), 100, 3), full)
    # with blocks of 3 and a window of 7, position 12 sees tokens 6..12 and the blocks 0 and 1 (tokens 0..5)
    keys = torch.cat([k[:6, 0].reshape(2, 3, 6).mean(1), k[6:13, 0]])
    vals = torch.cat([v[:6, 0].reshape(2, 3, 5).mean(1), v[6:13, 0]])
    want = torch.softmax(keys @ q[12, 1] * 0.4, 0) @ vals
    assert torch.allclose(O.pooled_window_attention(q, k, v, torch.full((4,), 0.4, dtype=F64), 7, 3)[12, 1], want)
    # position 11: token 5 has left the window, its block (3..5) ends at 5 > 11 - 7: only block 0 is seen
    keys = torch.cat([k[:3, 0].mean(0, keepdim=True), k[5:12, 0]])
    vals = torch.cat([v[:3, 0].mean(0, keepdim=True), v[5:12, 0]])
    want = torch.softmax(keys @ q[11, 0] * 0.4, 0) @ vals
    assert torch.allclose(O.pooled_window_attention(q, k, v, torch.full((4,), 0.4, dtype=F64), 7, 3)[11, 0], want)
    # rotations keep the norm, act on the leading entries only, and the layouts pair different entries
    x = r(9, 2, 10)
    pos = torch.arange(9)
    for layout in ("half", "interleaved"):
        y = O.rotate(x, pos, 100.0, 6, layout)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1)) and torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    assert not torch.allclose(O.rotate(x, pos, 100.0, 6, "half"), O.rotate(x, pos, 100.0, 6, "interleaved"))
    # the diagonal recurrence with closed gates keeps nothing of the input: a = exp(-8 r softplus(lam)) -> S stays 0 for i = 0
    W = {"ra": torch.zeros(1, 4, 4, dtype=F64), "ri": torch.zeros(1, 4, 4, dtype=F64), "ra.b": torch.zeros(1, 4, dtype=F64),
         "ri.b": torch.full((1, 4), -50.0, dtype=F64), "lam": torch.zeros(4, dtype=F64)}
    assert float(O.gated_diagonal_recurrence(r(12, 4), W, 1).abs().max()) < 1e-12
    # ... and with an open input gate the state is a normalised moving average with a = exp(-4 ln 2)
    W["ri.b"] = torch.full((1, 4), 50.0, dtype=F64)
    u = r(12, 4)
    a = 2.0 ** -4
    S = torch.zeros(4, dtype=F64)
    for t in range(12):
        S = a * S + (1 - a * a) ** 0.5 * u[t]
    assert torch.allclose(O.gated_diagonal_recurrence(u, W, 1)[-1], S)
    # the clamped feed-forward: limits bite on the gate from above only, on the other branch from both sides
    h = torch.eye(3, dtype=F64) * 100.0
    ffw = {"gate": torch.tensor([[1.0, 0, 0], [0, -1.0, 0]], dtype=F64), "up": torch.tensor([[0, 0, 1.0], [0, 0, -1.0]], dtype=F64),
           "down": torch.eye(2, dtype=F64)}
    y = O.clamped_gated_ff(h, ffw, 2.0)
    assert torch.allclose(y[0], torch.tensor([2.0 * torch.sigmoid(torch.tensor(3.404, dtype=F64)), 0.0], dtype=F64))
    assert float(y[1].abs().max()) < 1e-30                 # a gate of -100 is not clamped from below: g sigmoid(1.702 g) vanishes
    # whole model: a prefix's logits do not depend on what follows
    d = _cfg()
    Wm = O.random_weights(d, seed=4)
    toks = torch.randint(0, 131, (30,), generator=g).tolist()
    full = O.forward(d, Wm, toks)
    assert torch.allclose(O.forward(d, Wm, toks[:17]), full[:17], atol=1e-9)
