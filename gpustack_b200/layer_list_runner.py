"""Model runner of the layer-list decoders (config.LayerListConfig: Vodavik, Danipel, Resevik, Dotorax).

Same step interface as runner.ModelRunner -- the engine, the scheduler's plans, the staging buffer, CUDA-graph
decode steps and the sampler are shared -- with this family's layer sequence:

    embed -> per layer [ fused input projection -> mixer -> output projection -> LN(alpha x + y)
                         ( -> up projection -> relu^2 -> down projection -> LN(alpha x + y) ) ]
          -> final LN of the wanted rows (x logit_scale) -> lm_head (fp32 logits) -> sampler

  attention mixer: attn_prep (bias, q/k head norms, query temperature, K/V page scatter) -> sink-softmax
                   attention over the paged cache (prefill tiles for prompt portions, the decode kernel for
                   single new rows; both in one mixed step) with the sigmoid output gate in its epilogue;
                   a `kv_from` layer skips the scatter and reads the owner layer's pages.
  mlstm mixer:     fp32 gate projection -> matrix-memory scan over every sequence's new rows (state slot in /
                   out, fp32) -> per-head unit RMS x norm weight x sigmoid gate.

  latent_attention mixer: fused projection [q or query latent | latent | key part] (-> RMS norm -> query
                   up-projection) -> latent_prep (latent norm + rotated key part into the token's ONE cache row,
                   rotated query parts) -> per-head absorption of W_uk into the query -> attention over the latent
                   cache (one shared row per token: G = 1, values = the first kv_rank entries of the key rows;
                   softmax sink optional) -> per-head W_uv -> output projection.

  linear_attention mixer: rot_prep (feature map / rotation / key factor -> fp32 q | k | v rows) -> decayed
                   linear-attention scan over every sequence's new rows (state slot in / out, fp32; chunk form for
                   prompt portions) -> output norm (per head, or all heads with a weight) x sigmoid / SiLU gate.
  attention mixer with rotation: rot_prep (rotation, weightless q / k norm, keys to their pages, values = the keys
                   as projected) -> the same attention kernels, with a sliding window.

Residual schemes (config.residual): "post_ln" as drawn above; "parallel": pre-norm with ONE RMS norm per layer,

    embed * scale -> per layer run [ x += branches of the layer before (+ embedding before a repeated pass) ; h = RMSnorm(x)
                                     -> mixer(h) and feed-forward(h) side by side ] -> x += last branches -> RMSnorm

where a span of layers may run several times with the same weights (config.runs(): caches and state per run) and
ONE add_rms_norm launch does the sum and the next norm; "streams": pre-norm over S fp32 residual copies,

    embed * scale -> S streams -> per sublayer [ u = sum_s in[s] x_s -> tanh norm -> sublayer ->
                                                 x_t <- sum_s mix[s,t] x_s + m out[t] y ]  -> sum of the streams -> tanh norm

where ONE streams_step launch does a sublayer's write-back and the next sublayer's read + norm.  "sandwich": a norm before AND after every sublayer,

    embed + learned position -> per sublayer [ x += m * norm_b(output of the sublayer before) ; h = norm_a(x)
                                               -> h + causal conv(h) (ring of the last inputs per sequence) -> sublayer ]
          -> x += m * norm_b(last output) -> norm of the wanted rows

where ONE sandwich_join launch does the sum (with the post-norm of the output) and the next pre-norm, and the short
convolution with its per-sequence ring follows.  Its mixers: rotary attention with one gate per head; a side-by-side
pair of [sliding-window attention that also sees the pooled blocks before the window | gated diagonal recurrence behind a
short convolution], whose two output projections meet in the join with their factors; gated linear attention with a
decay per key channel and token.

Feed-forwards:
relu^2 (ungated), gated GELU, a clamped gated unit, or a routed mixture of clamped gated experts with identity experts
and a shared expert (ops.routed_experts).

The residual stream is fp32 from the embedding to the final norm, and so is every sublayer's output on its way
into the sum (the output projections write fp32); projections read a copy of the stream rounded once to bf16.  With EngineConfig.dtype == "float32" every activation, cache and product is fp32 (CUDA-core GEMM with
FMA accumulation: no TF32, no bf16 anywhere but the stored weights, which convert exactly).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import ops
from .lib import B200Error
from .runner import BF16, ModelRunner


class LayerListRunner(ModelRunner):
    SUPPORTS_FP32 = True

    # ------------------------------------------------------------------------------ memory
    def _init_model_dims(self):
        cfg = self.mcfg
        if self.tp != 1:
            raise B200Error("layer-list models run with tensor_parallel_size=1")
        self.act_dtype = torch.float32 if self.ecfg.dtype == "float32" else BF16
        self.fp8 = False
        # attention layers whose keys and values have one tile-sized width run on the tensor-core kernels of the
        # Llama-class models (extended with the sink and the gate); the others on the generic kernels
        bf = self.act_dtype == BF16
        attn = [(l, x.mixer.left if x.mixer.kind == "side_by_side" else x.mixer) for l, x in enumerate(cfg.layers)
                if x.mixer.kind in ("attention", "side_by_side")]
        self.fast_decode = {l: bf and m.tile_sized for l, m in attn}
        self.fast_prefill = {l: bf and m.tile_sized and ops.attn_prefill_tc_covers(m.heads, m.kv_heads, m.dim) for l, m in attn}
        base = ops.attn_sink_prefill_tile()
        # ONE tile list serves every layer of a step: the tile size most tensor-core layers want (ties: the larger)
        tiles = [ops.attn_prefill_tile(m.heads, m.kv_heads) for l, m in attn
                 if self.fast_prefill[l] or (bf and m.pool and m.dim == m.vdim and ops.attn_prefill_tc_covers(m.heads, m.kv_heads, m.dim))]
        self.prefill_tile = max(set(tiles), key=lambda t: (tiles.count(t), t)) if tiles else base
        for l, m in attn:
            if self.fast_prefill[l] and ops.attn_prefill_tile(m.heads, m.kv_heads) != self.prefill_tile:
                self.fast_prefill[l] = False
        # a window with pooled blocks: the window's tokens on the tcgen05 kernel (which hands over every row's log-sum-exp),
        # the pooled blocks by the generic kernel that continues that softmax
        self.pool_tc = {l: bool(bf and ops.LAYER_LIST_TC and m.pool and m.dim == m.vdim and ops.attn_prefill_tc_covers(m.heads, m.kv_heads, m.dim)
                                and ops.attn_prefill_tile(m.heads, m.kv_heads) == self.prefill_tile) for l, m in attn}
        # ... and single rows on the split-KV decode kernel in the same way
        self.pool_dec = {l: bool(bf and ops.LAYER_LIST_TC and m.pool and m.tokens_tile_sized) for l, m in attn}
        if self.prefill_tile % base:
            raise B200Error("prefill tile sizes of the attention kernels do not nest")
        self._dec_ws = {}
        self.streams = cfg.residual == "streams"
        self.parallel = cfg.residual == "parallel"
        self.sandwich = cfg.residual == "sandwich"
        self.canon_taps = getattr(cfg, "canon_taps", 0)
        self.runs = cfg.runs()                 # [(layer, embedding added before it)]: caches and state belong to a run
        self.looped = any(again for _, again in self.runs)
        self.layer_trace = None                # a list: receives the fp32 residual after every layer run (tests, debugging)
        self.S = cfg.n_streams if self.streams else 1
        self.proj_width = max(lw.proj.shape[0] for lw in self.w.layers)
        self.mix_width = max(l.mixer.out_width for l in cfg.layers)
        self.ff_width = max([(l.mlp.moe.shared_ff if l.mlp.kind == "moe" else l.mlp.ff) for l in cfg.layers
                             if l.mlp is not None] or [0])
        lat = [l.mixer for l in cfg.layers if l.mixer.kind == "latent_attention"]
        self.lat_q_width = max([m.q_width for m in lat if m.q_rank] or [0])
        self.lat_q_rank = max([m.q_rank for m in lat] or [0])
        self.lat_qa_width = max([m.heads * m.cache_width for m in lat] or [0])
        self.lat_o_width = max([m.heads * m.kv_rank for m in lat] or [0])
        self.routed = [l.mlp.moe for l in cfg.layers if l.mlp is not None and l.mlp.kind == "moe"]
        rec = [l.mixer for l in cfg.layers if l.mixer.kind == "mlstm"]
        lin = [l.mixer for l in cfg.layers if l.mixer.kind in ("linear_attention", "gated_linear_attention")]
        gla = [l.mixer for l in cfg.layers if l.mixer.kind == "gated_linear_attention"]
        gdr = [l.mixer.right for l in cfg.layers if l.mixer.kind == "side_by_side"]
        # (a side-by-side mixer's attention also parks its rows' log-sum-exp here, one number per head)
        self.gate_width = max([2 * m.heads for m in rec] + [m.heads * m.dim for m in gla] + [2 * m.width for m in gdr]
                              + [l.mixer.left.heads for l in cfg.layers if l.mixer.kind == "side_by_side"] or [0])
        self.rec_width = max([m.out_width for m in rec + lin] or [0])
        self.lin_width = max([2 * m.heads * m.dim + m.out_width for m in lin] + [m.width for m in gdr] or [0])
        self.state: List[Optional[tuple]] = [None] * len(self.runs)
        self.canon_ring: List[Optional[tuple]] = [None] * len(self.runs)   # input-convolution rings (mixer, feed-forward) per run
        self.pool_k: List[Optional[torch.Tensor]] = [None] * len(self.runs)
        self.pool_v: List[Optional[torch.Tensor]] = [None] * len(self.runs)
        self.num_state_slots = 0

    def _alloc_model_buffers(self):
        dev, T, D = self.device, self.max_tokens, self.H
        e = lambda *s, dt: torch.empty(*s, dtype=dt, device=dev)   # noqa: E731
        a = self.act_dtype
        self.resid32 = e(T, self.S * D, dt=torch.float32)  # the residual stream (S copies per row with hyper-connections)
        self.xb = e(T, D, dt=a)                           # the same rows as the projections read them
        self.y = e(T, D, dt=torch.float32)                # a sublayer's output: fp32 into the residual sum
        self.proj = e(T * self.proj_width, dt=a)          # flat; viewed [T, rows of this layer's fused projection]
        self.mix_out = e(T * self.mix_width, dt=a)
        self.act = e(T * max(1, self.ff_width), dt=a)
        self.gates = e(T * max(1, self.gate_width), dt=torch.float32)
        self.o_raw = e(T * max(1, self.rec_width), dt=torch.float32)
        self.lin32 = e(T * max(1, self.lin_width), dt=torch.float32)   # prepared q | k | v rows of a linear-attention mixer
        gdr = [l.mixer.right.width for l in self.mcfg.layers if l.mixer.kind == "side_by_side"]
        self.rec_ws = ops.gated_recurrence_workspace(T, self.max_seqs, max(gdr), dev) if gdr else None
        if self.sandwich:
            self.y2 = e(T, D, dt=torch.float32)           # the second output of a side-by-side mixer
            self.h32 = e(T, D, dt=torch.float32)          # a sublayer's normed input before its convolution
        if self.parallel:
            self.y2 = e(T, D, dt=torch.float32)           # the feed-forward's output beside the mixer's (self.y)
            self.emb32 = e(T, D, dt=torch.float32) if self.looped else None   # the embedding output, added again per pass
        self._pending = (None, None)                      # branch outputs not yet summed into the residual
        self.lat_q = e(T * max(1, self.lat_q_width), dt=a)        # queries of a mixer whose queries have a latent
        self.lat_cq = e(T * max(1, self.lat_q_rank), dt=a)        # the normed query latent
        self.lat_qa = e(T * max(1, self.lat_qa_width), dt=a)      # absorbed queries [H][kv_rank | rot_dim]
        self.lat_o = e(T * max(1, self.lat_o_width), dt=a)        # attention output in latent space [H][kv_rank]
        self.routed_ws = None
        if self.routed:
            self.routed_ws = ops.RoutedWorkspace(T, max(r.top for r in self.routed),
                                                 max(r.experts + r.identity for r in self.routed), D,
                                                 max(r.ff for r in self.routed), a, dev)

    def _alloc_step_io(self):
        super()._alloc_step_io()
        self.x_last = torch.empty(self.max_sample, self.H, dtype=self.act_dtype, device=self.device)

    def kv_block_bytes(self) -> int:
        return self.block_size * self.mcfg.kv_bytes_per_token(elem_bytes=4 if self.act_dtype == torch.float32 else 2)

    def init_kv_cache(self, num_blocks: int) -> None:
        """Pages of every attention layer that owns keys and values; a `kv_from` layer aliases its owner's."""
        self.num_blocks = num_blocks
        cfg = self.mcfg
        self.k_cache = [None] * len(self.runs)
        self.v_cache = [None] * len(self.runs)
        for l, (li, _) in enumerate(self.runs):          # one cache per RUN of a layer (a repeated span: one per pass)
            m = cfg.layers[li].mixer
            if m.kind == "side_by_side":
                m = m.left
                per_page = m.pool_per_page(self.block_size)
                # mean key / value of every block of m.pool tokens, fp32, addressed through the KV block table
                self.pool_k[l] = torch.zeros(num_blocks, m.kv_heads, per_page, m.dim, dtype=torch.float32, device=self.device)
                self.pool_v[l] = torch.zeros(num_blocks, m.kv_heads, per_page, m.vdim, dtype=torch.float32, device=self.device)
            if m.kind == "attention" and m.kv_from is None:
                self.k_cache[l] = torch.zeros(num_blocks, m.kv_heads, self.block_size, m.dim, dtype=self.act_dtype,
                                              device=self.device)
                self.v_cache[l] = torch.zeros(num_blocks, m.kv_heads, self.block_size, m.vdim, dtype=self.act_dtype,
                                              device=self.device)
            elif m.kind == "latent_attention":
                # ONE row per token for all heads: [latent: kv_rank | rotated key part: rot_dim]; the values are its head
                self.k_cache[l] = torch.zeros(num_blocks, 1, self.block_size, m.cache_width, dtype=self.act_dtype,
                                              device=self.device)
                self.v_cache[l] = self.k_cache[l]
        for l, (li, _) in enumerate(self.runs):
            m = cfg.layers[li].mixer
            if m.kind == "attention" and m.kv_from is not None:      # (designs with kv_from have no repeated span)
                self.k_cache[l], self.v_cache[l] = self.k_cache[m.kv_from], self.v_cache[m.kv_from]

    def init_state(self, num_slots: int) -> None:
        """fp32 recurrent state of every mlstm layer for `num_slots` sequences (kv_cache.StateSlotPool hands
        the slots out): S [slots, H, dv, dk] (key index fastest), and per 32-column slice of dv the normaliser n [slots, H, Z, dk]
        and the stabiliser m [slots, H, Z]."""
        self.num_state_slots = num_slots
        f = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)   # noqa: E731
        D, R = self.H, self.canon_taps - 1
        for l, (li, _) in enumerate(self.runs):
            m = self.mcfg.layers[li].mixer
            if R > 0:        # the last inputs of the mixer's and the feed-forward's convolution, by position mod R
                self.canon_ring[l] = (f(num_slots, R, D), f(num_slots, R, D) if self.mcfg.layers[li].mlp is not None else None)
            if m.kind == "side_by_side":             # S [slots, W], and the ring of its convolution's last inputs
                r = m.right
                self.state[l] = (f(num_slots, r.width), f(num_slots, r.conv - 1, r.width) if r.conv > 1 else None)
            if m.kind in ("linear_attention", "gated_linear_attention"):         # S [slots, H, dv, dk]
                self.state[l] = (f(num_slots, m.heads, m.vdim, m.dim),)
            if m.kind != "mlstm":
                continue
            z = ops.mlstm_state_slices(m.vdim)
            self.state[l] = (f(num_slots, m.heads, m.vdim, m.dim), f(num_slots, m.heads, z, m.dim), f(num_slots, m.heads, z))

    def init_host_kv(self, slots: int) -> None:
        self.host_slots = 0          # no prefix reuse with recurrent state: nothing to keep on the host

    # ------------------------------------------------------------------------------ layers
    def _view(self, buf: torch.Tensor, T: int, n: int) -> torch.Tensor:
        return buf[:T * n].view(T, n)

    def _embed(self, ids: torch.Tensor, T: int) -> None:
        if self.streams:
            lw = self.w.layers[0]
            ops.embed_streams(ids, self.w.embed, self.resid32[:T], self.S, self.mcfg.embed_scale)
            ops.streams_step(self.resid32[:T], self.S, hc_read=lw.hc1, norm=(lw.norm1_alpha, lw.norm1, lw.norm1_b),
                             xb_out=self.xb[:T])
            self.stats["kernel_launches"] += 2
            return
        if self.sandwich:
            if self.mcfg.learned_positions:
                ops.embed_pos(ids, self._pos[:T], self.w.embed, self.w.pos, self.resid32[:T])
            else:
                ops.embed_streams(ids, self.w.embed, self.resid32[:T], 1, self.mcfg.embed_scale)
            self._pending = None
            self.stats["kernel_launches"] += 1
            return
        if self.parallel:      # the first layer's norm reads the embedding output; a repeated span adds it again
            ops.embed_streams(ids, self.w.embed, self.emb32[:T] if self.looped else self.resid32[:T], 1,
                              self.mcfg.embed_scale)
            self._pending = (None, None)
            self.stats["kernel_launches"] += 1
            return
        ops.embed_rows(ids, self.w.embed, self.resid32[:T], self.xb[:T])
        self.stats["kernel_launches"] += 1

    def _open_layer(self, T: int, r: int, lw, again: bool) -> None:
        """Parallel residual: the branch outputs of the layer before (and, before a repeated pass, the embedding
        output) enter the fp32 stream, and this layer's ONE norm prepares self.xb for its mixer and feed-forward."""
        a, b = self._pending
        first = r == 0 and self.looped
        ops.add_rms_norm(self.emb32[:T] if first else self.resid32[:T], lw.norm1, self.mcfg.norm_eps, a=a, b=b,
                         c=self.emb32[:T] if again else None, x_out=self.resid32[:T], xb_out=self.xb[:T])
        self._pending = (None, None)
        self.stats["kernel_launches"] += 1

    def _close_layer(self, T: int, has_ff: bool) -> None:
        self._pending = (self.y[:T], self.y2[:T] if has_ff else None)
        if self.layer_trace is not None:       # materialise the stream after this layer (not on the serving path)
            ops.add_rms_norm(self.resid32[:T], None, self.mcfg.norm_eps, a=self._pending[0], b=self._pending[1],
                             x_out=self.resid32[:T])
            self._pending = (None, None)
            self.layer_trace.append(self.resid32[:T].clone())

    def _sandwich_open(self, T: int, pre_w, conv_w, ring, cu_all, ctx_all, slots_all) -> None:
        """Sandwich residual: the output of the sublayer before (self._pending = (y, y2, ya, yb, post-norm weight))
        enters the fp32 stream through its norm, the stream is normed for the next sublayer, and the sublayer's input
        convolution (with the sequences' rings) prepares self.xb."""
        cfg = self.mcfg
        y, y2, ya, yb, post_w = self._pending if self._pending is not None else (None, None, 1.0, 1.0, None)
        h = self.h32[:T] if conv_w is not None else self.xb[:T]
        ops.sandwich_join(self.resid32[:T], cfg.norm_eps, y=y, y2=y2, ya=ya, yb=yb, post_w=post_w, mult=cfg.residual_mult,
                          pre_w=pre_w, x_out=self.resid32[:T] if y is not None else None, h_out=h)
        self._pending = None
        self.stats["kernel_launches"] += 1
        if conv_w is not None:
            ops.causal_conv(h, conv_w, ring, cu_all, ctx_all, slots_all, self.xb[:T], add_input=True)
            if ring is not None:
                ops.conv_commit(h, ring, cu_all, ctx_all, slots_all, conv_w.shape[1])
            self.stats["kernel_launches"] += 2

    def _sandwich_close(self, T: int) -> None:
        """Materialise the stream after a layer (tracing only: on the serving path the next sublayer's open does it)."""
        if self.layer_trace is None:
            return
        cfg = self.mcfg
        y, y2, ya, yb, post_w = self._pending
        ops.sandwich_join(self.resid32[:T], cfg.norm_eps, y=y, y2=y2, ya=ya, yb=yb, post_w=post_w, mult=cfg.residual_mult,
                          x_out=self.resid32[:T])
        self._pending = None
        self.layer_trace.append(self.resid32[:T].clone())

    def _join(self, T: int, l: int, q: int) -> None:
        """The branch output self.y of sublayer q (1 mixer, 2 feed-forward) of layer l enters the residual, and the
        next sublayer's input is prepared in self.xb."""
        cfg, lw = self.mcfg, self.w.layers[l]
        if not self.streams:
            self._post(T, lw.norm1 if q == 1 else lw.norm2)
            self.stats["kernel_launches"] += 1
            return
        if q == 1 and cfg.layers[l].mlp is not None:
            nxt = (lw.hc2, (lw.norm2_alpha, lw.norm2, lw.norm2_b))
        elif l + 1 < len(cfg.layers):
            n = self.w.layers[l + 1]
            nxt = (n.hc1, (n.norm1_alpha, n.norm1, n.norm1_b))
        else:
            nxt = (None, None)          # the last sublayer: the final norm runs on the wanted rows only
        ops.streams_step(self.resid32[:T], self.S, y=self.y[:T], hc_write=lw.hc1 if q == 1 else lw.hc2,
                         mult=cfg.residual_mult, hc_read=nxt[0], norm=nxt[1], xb_out=self.xb[:T] if nxt[1] else None)
        self.stats["kernel_launches"] += 1

    def _post(self, T: int, norm_w: torch.Tensor) -> None:
        cfg = self.mcfg
        ops.sum_layer_norm(self.y[:T], self.resid32[:T], norm_w, cfg.postln_alpha, cfg.norm_eps,
                           x_out=self.resid32[:T], xb_out=self.xb[:T])

    def _decode_plan(self, B: int, m):
        """(KV splits, workspace) of the split-KV decode kernel for B rows of mixer m; one zero-initialised,
        self-resetting workspace per head shape, sized for the largest batch."""
        span = min(self.max_model_len, m.window) if m.window else self.max_model_len    # keys a row can see
        splits = ops.attn_decode_splits(B, m.kv_heads, span)
        key = (m.heads, m.kv_heads, m.dim, span)
        if key not in self._dec_ws:
            from .lib import load

            L = load()
            need = max(L.b200_attn_decode_workspace_bytes(b, m.heads, m.dim, ops.attn_decode_splits(b, m.kv_heads, span))
                       for b in range(1, self.max_seqs + 1))
            self._dec_ws[key] = torch.zeros((need + 3) // 4, dtype=torch.float32, device=self.device)
        return splits, self._dec_ws[key]

    def _latent_decode_plan(self, B: int, m):
        """(key ranges, workspace) of the latent decode attention for B rows of mixer m; one workspace per shape, sized
        for the largest batch and the most ranges."""
        if self.act_dtype != BF16 or not ops.latent_attn_covers(m.heads, m.kv_rank, m.rot_dim):
            return 1, None
        splits = ops.latent_attn_decode_splits(B, m.heads, self.max_model_len)
        key = ("latent", m.heads, m.kv_rank)
        if key not in self._dec_ws:
            self._dec_ws[key] = ops.latent_attn_decode_workspace(self.max_seqs, m.heads, m.kv_rank, 16, self.device)
        return splits, self._dec_ws[key]

    def _run_layers(self, T: int, Tp: int, Bd: int, nt: int, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d, cu_all, ctx_all,
                    slots_all) -> None:
        """Rows [0, Tp): prompt portions (tiles ts / tq over cu_p / ctx_p / bt_p); rows [Tp, T): Bd single new
        rows (lens_d / bt_d).  cu_all / ctx_all / slots_all list both kinds for the recurrent scan."""
        cfg, eps = self.mcfg, self.mcfg.norm_eps
        pos, slots = self._pos, self._slots
        for l, (li, again) in enumerate(self.runs):      # l indexes the run (caches, state), li the layer (weights)
            layer, lw = cfg.layers[li], self.w.layers[li]
            m = layer.mixer
            proj = self._view(self.proj, T, lw.proj.shape[0])
            out = self._view(self.mix_out, T, m.out_width)
            if self.parallel:
                self._open_layer(T, l, lw, again)
            if self.sandwich:
                ring = self.canon_ring[l] or (None, None)
                self._sandwich_open(T, lw.norm1, lw.canon1, ring[0], cu_all, ctx_all, slots_all)
            ops.linear(self.xb[:T], lw.proj, proj)
            if m.kind == "side_by_side":
                self._side_by_side(l, m, lw, proj, out, T, Tp, Bd, nt, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d, cu_all, ctx_all,
                                   slots_all)
                if layer.mlp is not None:
                    self._sandwich_open(T, lw.norm2, lw.canon2, ring[1], cu_all, ctx_all, slots_all)
                    self._feed_forward(T, layer.mlp, lw)
                    self._pending = (self.y[:T], None, 1.0, 1.0, lw.norm2b)
                self._sandwich_close(T)
                continue
            if m.kind == "gated_linear_attention":
                H, dk, dv = m.heads, m.dim, m.vdim
                kc, vc = H * dk, 2 * H * dk
                gc = vc + H * dv
                ac = gc + H * dv
                x32 = self._view(self.lin32, T, gc)
                # q / sqrt(dk), k, v as fp32 rows; the decay's pre-activation z = A2 (A1 h) + b in fp32
                ops.rot_prep(proj, 0, kc, vc, pos, None, x32, x32[:, kc:], x32[:, vc:], H, H, dk, dv, paged=False,
                             q_mul=dk ** -0.5)
                z = self._view(self.gates, T, kc)
                ops.linear(proj[:, ac:ac + m.decay_rank], lw.decay_up, z, bias=lw.decay_bias)
                o_raw = self._view(self.o_raw, T, H * dv)
                ops.gla_scan(x32, 0, kc, vc, z, 1.0 / m.tau, cu_all, ctx_all, slots_all, self.state[l][0], o_raw, H, dk, dv,
                             max_len=Tp if Tp else 1)
                ops.linattn_out(o_raw, proj, gc, lw.out_norm, out, H, dv, eps, False, "silu")
                self.stats["kernel_launches"] += 5
            elif m.kind == "latent_attention":
                self._latent_attention(l, m, lw, proj, out, T, Tp, Bd, nt, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d)
            elif m.kind == "attention":
                own = m.kv_from is None
                H, G, dk, dv = m.heads, m.kv_heads, m.dim, m.vdim
                if m.rot is not None or m.values_are_keys or m.qk_unit_norm:
                    # rotation, then the weightless q / k norm; keys to their pages, values = the keys as projected
                    # (a layer that reads another layer's cache prepares its queries only)
                    ops.rot_prep(proj, 0, H * dk, -1 if m.values_are_keys else (H + G) * dk, pos, slots, proj,
                                 self.k_cache[l] if own else None, self.v_cache[l] if own else None, H, G, dk, dv, paged=True,
                                 rot_dims=m.rot.dims if m.rot is not None else 0,
                                 half_layout=m.rot is not None and m.rot.layout == "half", freq=lw.rot_freq,
                                 unit_norm=m.qk_unit_norm, eps=eps)
                else:
                    ops.attn_prep(proj, lw.proj_bias, lw.q_norm, lw.k_norm, pos, slots, self.k_cache[l] if own else None,
                                  self.v_cache[l] if own else None, H, G, dk, dv, eps, m.q_temp_coef, m.q_temp_every)
                kv_cols = 0 if not own else (G * dk if m.values_are_keys else G * (dk + dv))
                gate_col = (H * dk + kv_cols) if m.gate else -1
                kc, vc = self.k_cache[l], self.v_cache[l]
                if nt and self.fast_prefill[li]:
                    ops.paged_attn_prefill_ex(proj[:Tp], proj.stride(0), kc, vc, bt_p, cu_p, ctx_p, ts, tq, out[:Tp], H, G, dk,
                                              m.scale, sink=lw.sink, gate=proj[:Tp, gate_col:] if m.gate else None,
                                              window=m.window, gate_per_head=m.gate_per_head)
                elif nt:
                    ops.attn_sink_prefill(proj[:Tp], gate_col, kc, vc, bt_p, cu_p, ctx_p, ts, tq, lw.sink, out[:Tp],
                                          H, G, dk, dv, m.scale, tile_rows=self.prefill_tile, window=m.window,
                                          gate_per_head=m.gate_per_head, head_scale=lw.head_scale)
                if Bd and self.fast_decode[li]:
                    splits, ws = self._decode_plan(Bd, m)
                    ops.paged_attn_decode(proj[Tp:T], proj.stride(0), kc, vc, bt_d, lens_d, out[Tp:T], H, G, dk, m.scale,
                                          num_splits=splits, workspace=ws, sink=lw.sink,
                                          gate=proj[Tp:T, gate_col:] if m.gate else None, window=m.window,
                                          gate_per_head=m.gate_per_head)
                elif Bd:
                    ops.attn_sink_decode(proj[Tp:T], gate_col, kc, vc, bt_d, lens_d, lw.sink, out[Tp:T], H, G, dk, dv,
                                         m.scale, window=m.window, gate_per_head=m.gate_per_head, head_scale=lw.head_scale)
                self.stats["kernel_launches"] += 2 + (1 if nt else 0) + (1 if Bd else 0)
            elif m.kind == "linear_attention":
                H, dk, dv = m.heads, m.dim, m.vdim
                kc, vc = H * dk, 2 * H * dk
                x32 = self._view(self.lin32, T, vc + H * dv)
                # feature map / rotation / key factor in fp32: what enters the recurrence is never rounded to bf16
                ops.rot_prep(proj, 0, kc, vc, pos, None, x32, x32[:, kc:], x32[:, vc:], H, H, dk, dv, paged=False,
                             feature=m.feature, rot_dims=m.rot.dims if m.rot is not None else 0,
                             half_layout=m.rot is not None and m.rot.layout == "half", freq=lw.rot_freq, k_mul=m.k_scale)
                o_raw = self._view(self.o_raw, T, H * dv)
                ops.linattn_scan(x32, 0, kc, vc, lw.decay, cu_all, ctx_all, slots_all, self.state[l][0], o_raw, H, dk, dv,
                                 max_len=Tp if Tp else 1)
                ops.linattn_out(o_raw, proj, vc + H * dv, lw.out_norm, out, H, dv, eps, m.out_norm == "all_heads", m.gate_act)
                self.stats["kernel_launches"] += 4
            else:
                H, dk, dv = m.heads, m.dim, m.vdim
                gates = self._view(self.gates, T, 2 * H)
                ops.linear(self.xb[:T], lw.gates, gates)
                o_raw = self._view(self.o_raw, T, H * dv)
                S, n, mm = self.state[l]
                ops.mlstm_scan(proj, 0, H * dk, 2 * H * dk, gates, lw.gate_bias, cu_all, ctx_all, slots_all, S, n, mm,
                               o_raw, H, dk, dv, m.gate_cap, max_len=Tp if Tp else 1)
                ops.mlstm_out(o_raw, proj, 2 * H * dk + H * dv, lw.out_norm, out, H, dv, eps)
                self.stats["kernel_launches"] += 4
            ops.linear(out, lw.o, self.y[:T])
            self.stats["kernel_launches"] += 1
            if self.sandwich:
                self._pending = (self.y[:T], None, 1.0, 1.0, lw.norm1b)
                if layer.mlp is not None:
                    self._sandwich_open(T, lw.norm2, lw.canon2, ring[1], cu_all, ctx_all, slots_all)
                    self._feed_forward(T, layer.mlp, lw)
                    self._pending = (self.y[:T], None, 1.0, 1.0, lw.norm2b)
                self._sandwich_close(T)
                continue
            if self.parallel:      # the feed-forward reads the same normed rows; both outputs wait for the next norm
                if layer.mlp is not None:
                    self._feed_forward(T, layer.mlp, lw, self.y2[:T])
                self._close_layer(T, layer.mlp is not None)
                continue
            self._join(T, li, 1)
            if layer.mlp is not None:
                self._feed_forward(T, layer.mlp, lw)
                self._join(T, li, 2)

    def _side_by_side(self, l, m, lw, proj, out, T, Tp, Bd, nt, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d, cu_all, ctx_all,
                      slots_all) -> None:
        """Two mixers on one input.  Left: rotary attention in a sliding window that also sees the mean key / value of
        every block of tokens wholly before the window (block means kept in a second cache, refreshed for the blocks
        this step completes).  Right: [y | x] branches -> short convolution of x (ring per sequence) -> block-diagonal
        gate projections in fp32 -> the gated diagonal recurrence (state slot in / out) times gelu(y).  Each side has
        its own output projection (fp32); the join that follows mixes them with the mixer's factors."""
        a, r = m.left, m.right
        eps = self.mcfg.norm_eps
        H, G, dk, dv, W = a.heads, a.kv_heads, a.dim, a.vdim, r.width
        # the two sides' outputs, each contiguous (the tensor-core attention kernel writes whole rows of heads)
        left = self.mix_out[:T * a.out_width].view(T, a.out_width)
        right = self.mix_out[T * a.out_width:T * (a.out_width + W)].view(T, W)
        kc, vc = self.k_cache[l], self.v_cache[l]
        li = self.runs[l][0]
        tc, dec = nt and self.pool_tc.get(li, False), Bd and self.pool_dec.get(li, False)
        # the per-head temperature rides in the query (a layer with a tensor-core route: those kernels have one scale) or
        # in the kernel; which one is the layer's property, not the step's, so a row's logits do not depend on the batch
        qmul = self.pool_tc.get(li, False) or self.pool_dec.get(li, False)
        ops.rot_prep(proj, 0, H * dk, (H + G) * dk, self._pos, self._slots, proj, kc, vc, H, G, dk, dv, paged=True,
                     rot_dims=a.rot.dims, half_layout=a.rot.layout == "half", freq=lw.rot_freq, unit_norm=a.qk_unit_norm, eps=eps,
                     q_head_mul=lw.head_scale if (qmul and lw.head_scale is not None) else None)
        hs = None if qmul else lw.head_scale
        pool = None
        if a.pool:
            pool = (self.pool_k[l], self.pool_v[l], a.pool)
            if nt:
                ops.kv_pool_update(kc, vc, pool[0], pool[1], bt_p, cu_p, ctx_p, cu_p.shape[0] - 1, Tp, a.pool)
            if Bd:
                ops.kv_pool_update(kc, vc, pool[0], pool[1], bt_d, None, lens_d, Bd, 1, a.pool)
        if tc:
            lse = self._view(self.gates, Tp, H)
            ops.paged_attn_prefill_ex(proj[:Tp], proj.stride(0), kc, vc, bt_p, cu_p, ctx_p, ts, tq, left[:Tp], H, G, dk, a.scale,
                                      window=a.window, lse_out=lse)
            ops.attn_sink_prefill_more(proj[:Tp], kc, bt_p, cu_p, ctx_p, ts, tq, left[:Tp], lse, H, G, dk, dv, a.scale,
                                       self.prefill_tile, a.window, None, pool)
            self.stats["kernel_launches"] += 1
        elif nt:
            ops.attn_sink_prefill(proj[:Tp], -1, kc, vc, bt_p, cu_p, ctx_p, ts, tq, None, left[:Tp], H, G, dk, dv, a.scale,
                                  tile_rows=self.prefill_tile, window=a.window, head_scale=hs, pool=pool)
        if dec:
            splits, ws = self._decode_plan(Bd, a)
            lse = self._view(self.gates, T, H)[Tp:T]
            ops.paged_attn_decode(proj[Tp:T], proj.stride(0), kc, vc, bt_d, lens_d, left[Tp:T], H, G, dk, a.scale,
                                  num_splits=splits, workspace=ws, window=a.window, lse_out=lse)
            ops.attn_sink_decode_more(proj[Tp:T], kc, bt_d, lens_d, left[Tp:T], lse, H, G, dk, dv, a.scale, a.window, None, pool)
            self.stats["kernel_launches"] += 1
        elif Bd:
            ops.attn_sink_decode(proj[Tp:T], -1, kc, vc, bt_d, lens_d, None, left[Tp:T], H, G, dk, dv, a.scale,
                                 window=a.window, head_scale=hs, pool=pool)
        y_col = a.q_width + G * (dk + dv)
        x_in = proj[:, y_col + W:y_col + 2 * W]
        S, ring = self.state[l]
        u = self._view(self.lin32, T, W)
        ops.causal_conv(x_in, lw.rec_conv, ring, cu_all, ctx_all, slots_all, u, add_input=False, in_bias=lw.rec_bias[W:],
                        bias=lw.rec_conv_bias)
        if ring is not None:
            ops.conv_commit(x_in, ring, cu_all, ctx_all, slots_all, r.conv, in_bias=lw.rec_bias[W:])
        gates = self._view(self.gates, T, 2 * W)
        n = W // r.blocks
        ops.head_linear(u, lw.rec_gates[:r.blocks], gates[:, :W], r.blocks, n=n, k=n, x_head=n, out_head=n)
        ops.head_linear(u, lw.rec_gates[r.blocks:], gates[:, W:], r.blocks, n=n, k=n, x_head=n, out_head=n)
        ops.gated_recurrence_scan(u, gates, lw.rec_gate_bias, lw.rec_lam, proj, y_col, lw.rec_bias[:W], cu_all, ctx_all,
                                  slots_all, S, right, r.gate_c, max_len=Tp if Tp else 1, workspace=self.rec_ws)
        ops.linear(left, lw.o, self.y[:T])
        ops.linear(right, lw.o2, self.y2[:T])
        self._pending = (self.y[:T], self.y2[:T], m.left_scale, m.right_scale, lw.norm1b)
        self.stats["kernel_launches"] += 9 + (2 if nt else 0) + (2 if Bd else 0)

    def _latent_attention(self, l, m, lw, proj, out, T, Tp, Bd, nt, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d) -> None:
        """Latent attention in the absorbed form: scores and values are taken straight from the cached latent rows,
        W_uk is folded into the query before and W_uv applied to the latent-space output after the attention, so a
        head's keys and values are never expanded and every head reads the same cache row."""
        eps = self.mcfg.norm_eps
        H, dn, dr, R, dv = m.heads, m.dim, m.rot_dim, m.kv_rank, m.vdim
        W = R + dr
        if m.q_rank:
            cq = self._view(self.lat_cq, T, m.q_rank)
            ops.rms_rows(proj[:, :m.q_rank], lw.q_lat_norm, cq, eps)
            q = self._view(self.lat_q, T, m.q_width)
            ops.linear(cq, lw.uq, q)
            kv_col = m.q_rank
            self.stats["kernel_launches"] += 2
        else:
            q, kv_col = proj[:, :m.q_width], m.q_width
        qa = self._view(self.lat_qa, T, H * W)
        o_lat = self._view(self.lat_o, T, H * R)
        cache = self.k_cache[l]
        ops.latent_prep(proj, kv_col, q, lw.kv_norm, self._pos, self._slots, cache, qa, H, dn, dr, R, m.rot.dims,
                        m.rot.layout == "half", lw.rot_freq, lw.rot_mag, eps)
        ops.head_linear(q, lw.uk_t, qa, H, n=R, k=dn, x_head=dn + dr, out_head=W)
        if nt:
            ops.latent_attn_prefill(qa[:Tp], cache, bt_p, cu_p, ctx_p, ts, tq, lw.sink, o_lat[:Tp], H, R, dr, m.scale,
                                    tile_rows=self.prefill_tile)
        if Bd:
            splits, ws = self._latent_decode_plan(Bd, m)
            ops.latent_attn_decode(qa[Tp:T], cache, bt_d, lens_d, lw.sink, o_lat[Tp:T], H, R, dr, m.scale, num_splits=splits,
                                   workspace=ws)
        ops.head_linear(o_lat, lw.uv, out, H, n=dv, k=R, x_head=R, out_head=dv)
        self.stats["kernel_launches"] += 3 + (1 if nt else 0) + (1 if Bd else 0)

    def _feed_forward(self, T: int, mlp, lw, y=None) -> None:
        """self.xb[:T] -> y (fp32; self.y[:T] unless given)."""
        y = self.y[:T] if y is None else y
        if mlp.kind == "moe" and mlp.moe.weight_on == "input":
            e = mlp.moe
            ops.routed_experts(self.xb[:T], lw.router, lw.correction, lw.w13, lw.w2, self.routed_ws, y, e.experts, 0, e.top,
                               e.scale, e.ff, e.limit, sigmoid=e.score == "sigmoid", renormalize=e.renormalize,
                               weight_on="input", act=e.act)
            self.stats["kernel_launches"] += ops.ROUTED_LAUNCHES
            return
        if mlp.kind == "moe":
            e = mlp.moe
            shared = None
            if e.shared_ff:
                act = self._view(self.act, T, e.shared_ff)
                ops.gated_linear(self.xb[:T], lw.shared13, act, "clamped_swish", e.shared_limit)
                shared = self.routed_ws.shared[:T]
                ops.linear(act, lw.shared2, shared)
                self.stats["kernel_launches"] += 2
            ops.routed_experts(self.xb[:T], lw.router, lw.correction, lw.w13, lw.w2, self.routed_ws, y, e.experts,
                               e.identity, e.top, e.scale, e.ff, e.limit, shared=shared)
            self.stats["kernel_launches"] += ops.ROUTED_LAUNCHES
            return
        act = self._view(self.act, T, mlp.ff)
        if mlp.act == "relu2":
            ops.linear(self.xb[:T], lw.up, act, relu2=True)            # squared ReLU in the GEMM's epilogue
        else:
            ops.gated_linear(self.xb[:T], lw.gate_up, act, mlp.act, mlp.limit)
        ops.linear(act, lw.down, y)
        self.stats["kernel_launches"] += 2

    def _forward_decode(self, ids, B: int, bt, lens, state_slots) -> None:
        if self.mcfg.has_state and self.num_state_slots == 0:
            raise B200Error("init_state() must run before the first step of a model with recurrent mixers")
        self._embed(ids, B)
        self._run_layers(B, 0, B, 0, None, None, None, None, None, lens, bt, self.arange_dev[:B + 1], self._pos,
                         state_slots)

    def _forward_prefill(self, ids, T, Tp, Bd, nt, bt_d, cu_d, ctx_d, ts_d, tq_d, dl_d, dbt_d, cu_all, ctx_all,
                         slots_all) -> None:
        if self.mcfg.has_state and self.num_state_slots == 0:
            raise B200Error("init_state() must run before the first step of a model with recurrent mixers")
        self._embed(ids, T)
        self._run_layers(T, Tp, Bd, nt, bt_d, cu_d, ctx_d, ts_d, tq_d, dl_d, dbt_d, cu_all, ctx_all, slots_all)

    def _sample(self, n: int, rows, temps, seeds) -> None:
        """Final norm of the wanted rows (times the logit scale, before the one rounding), lm_head, sampler."""
        cfg = self.mcfg
        if rows is None:
            rows = self.arange_dev[:n]
        if self.sandwich:      # the last sublayer's output enters the sum here, for the wanted rows only
            y, y2, ya, yb, post_w = self._pending if self._pending is not None else (None, None, 1.0, 1.0, None)
            ops.sandwich_join(self.resid32, cfg.norm_eps, y=y, y2=y2, ya=ya, yb=yb, post_w=post_w, mult=cfg.residual_mult,
                              pre_w=self.w.final_norm, rows=rows, h_out=self.x_last[:n])
        elif self.parallel:      # the last layer's branch outputs enter the sum here, for the wanted rows only
            a, b = self._pending
            ops.add_rms_norm(self.resid32, self.w.final_norm, cfg.norm_eps, a=a, b=b, rows=rows, xb_out=self.x_last[:n])
        elif self.streams:       # sum of the streams, tanh norm
            ops.streams_step(self.resid32, self.S, rows=rows, xb_out=self.x_last[:n],
                             norm=(self.w.final_norm_alpha, self.w.final_norm, self.w.final_norm_b))
        else:
            ops.sum_layer_norm(None, self.resid32, self.w.final_norm, 1.0, cfg.norm_eps, xb_out=self.x_last[:n], rows=rows,
                               out_scale=cfg.logit_scale)
        lg = self.logits[:n]
        ops.linear(self.x_last[:n], self.w.lm_head, lg)
        ops.sample(lg, temps, seeds, out_idx=self.out_ids[:n])
        self.stats["kernel_launches"] += 3


def runner_class(mcfg):
    """The runner of a model config's family."""
    return LayerListRunner if getattr(mcfg, "family", "") == "layer_list" else ModelRunner
