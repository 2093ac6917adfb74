"""Model runner of the layer-list decoders (config.LayerListConfig: Vodavik).

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
        attn = [(l, x.mixer) for l, x in enumerate(cfg.layers) if x.mixer.kind == "attention"]
        self.fast_decode = {l: bf and m.tile_sized for l, m in attn}
        self.fast_prefill = {l: bf and m.tile_sized and ops.attn_prefill_tc_covers(m.heads, m.kv_heads, m.dim) for l, m in attn}
        base = ops.attn_sink_prefill_tile()
        # ONE tile list serves every layer of a step: the tile size most tensor-core layers want (ties: the larger)
        tiles = [ops.attn_prefill_tile(m.heads, m.kv_heads) for l, m in attn if self.fast_prefill[l]]
        self.prefill_tile = max(set(tiles), key=lambda t: (tiles.count(t), t)) if tiles else base
        for l, m in attn:
            if self.fast_prefill[l] and ops.attn_prefill_tile(m.heads, m.kv_heads) != self.prefill_tile:
                self.fast_prefill[l] = False
        if self.prefill_tile % base:
            raise B200Error("prefill tile sizes of the attention kernels do not nest")
        self._dec_ws = {}
        self.proj_width = max(lw.proj.shape[0] for lw in self.w.layers)
        self.mix_width = max(l.mixer.out_width for l in cfg.layers)
        self.ff_width = max([l.mlp.ff for l in cfg.layers if l.mlp is not None] or [0])
        rec = [l.mixer for l in cfg.layers if l.mixer.kind == "mlstm"]
        self.gate_width = max([2 * m.heads for m in rec] or [0])
        self.rec_width = max([m.out_width for m in rec] or [0])
        self.state: List[Optional[tuple]] = [None] * len(cfg.layers)
        self.num_state_slots = 0

    def _alloc_model_buffers(self):
        dev, T, D = self.device, self.max_tokens, self.H
        e = lambda *s, dt: torch.empty(*s, dtype=dt, device=dev)   # noqa: E731
        a = self.act_dtype
        self.resid32 = e(T, D, dt=torch.float32)          # the residual stream
        self.xb = e(T, D, dt=a)                           # the same rows as the projections read them
        self.y = e(T, D, dt=torch.float32)                # a sublayer's output: fp32 into the residual sum
        self.proj = e(T * self.proj_width, dt=a)          # flat; viewed [T, rows of this layer's fused projection]
        self.mix_out = e(T * self.mix_width, dt=a)
        self.act = e(T * max(1, self.ff_width), dt=a)
        self.gates = e(T * max(1, self.gate_width), dt=torch.float32)
        self.o_raw = e(T * max(1, self.rec_width), dt=torch.float32)

    def _alloc_step_io(self):
        super()._alloc_step_io()
        self.x_last = torch.empty(self.max_sample, self.H, dtype=self.act_dtype, device=self.device)

    def kv_block_bytes(self) -> int:
        return self.block_size * self.mcfg.kv_bytes_per_token(elem_bytes=4 if self.act_dtype == torch.float32 else 2)

    def init_kv_cache(self, num_blocks: int) -> None:
        """Pages of every attention layer that owns keys and values; a `kv_from` layer aliases its owner's."""
        self.num_blocks = num_blocks
        cfg = self.mcfg
        self.k_cache = [None] * len(cfg.layers)
        self.v_cache = [None] * len(cfg.layers)
        for l, layer in enumerate(cfg.layers):
            m = layer.mixer
            if m.kind == "attention" and m.kv_from is None:
                self.k_cache[l] = torch.zeros(num_blocks, m.kv_heads, self.block_size, m.dim, dtype=self.act_dtype,
                                              device=self.device)
                self.v_cache[l] = torch.zeros(num_blocks, m.kv_heads, self.block_size, m.vdim, dtype=self.act_dtype,
                                              device=self.device)
        for l, layer in enumerate(cfg.layers):
            m = layer.mixer
            if m.kind == "attention" and m.kv_from is not None:
                self.k_cache[l], self.v_cache[l] = self.k_cache[m.kv_from], self.v_cache[m.kv_from]

    def init_state(self, num_slots: int) -> None:
        """fp32 recurrent state of every mlstm layer for `num_slots` sequences (kv_cache.StateSlotPool hands
        the slots out): S [slots, H, dv, dk] (key index fastest), and per 32-column slice of dv the normaliser n [slots, H, Z, dk]
        and the stabiliser m [slots, H, Z]."""
        self.num_state_slots = num_slots
        for l, layer in enumerate(self.mcfg.layers):
            m = layer.mixer
            if m.kind != "mlstm":
                continue
            z = ops.mlstm_state_slices(m.vdim)
            f = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)   # noqa: E731
            self.state[l] = (f(num_slots, m.heads, m.vdim, m.dim), f(num_slots, m.heads, z, m.dim), f(num_slots, m.heads, z))

    def init_host_kv(self, slots: int) -> None:
        self.host_slots = 0          # no prefix reuse with recurrent state: nothing to keep on the host

    # ------------------------------------------------------------------------------ layers
    def _view(self, buf: torch.Tensor, T: int, n: int) -> torch.Tensor:
        return buf[:T * n].view(T, n)

    def _embed(self, ids: torch.Tensor, T: int) -> None:
        ops.embed_rows(ids, self.w.embed, self.resid32[:T], self.xb[:T])
        self.stats["kernel_launches"] += 1

    def _post(self, T: int, norm_w: torch.Tensor) -> None:
        cfg = self.mcfg
        ops.sum_layer_norm(self.y[:T], self.resid32[:T], norm_w, cfg.postln_alpha, cfg.norm_eps,
                           x_out=self.resid32[:T], xb_out=self.xb[:T])

    def _decode_plan(self, B: int, m):
        """(KV splits, workspace) of the split-KV decode kernel for B rows of mixer m; one zero-initialised,
        self-resetting workspace per head shape, sized for the largest batch."""
        splits = ops.attn_decode_splits(B, m.kv_heads, self.max_model_len)
        key = (m.heads, m.kv_heads, m.dim)
        if key not in self._dec_ws:
            from .lib import load

            L = load()
            need = max(L.b200_attn_decode_workspace_bytes(b, m.heads, m.dim, ops.attn_decode_splits(b, m.kv_heads, self.max_model_len))
                       for b in range(1, self.max_seqs + 1))
            self._dec_ws[key] = torch.zeros((need + 3) // 4, dtype=torch.float32, device=self.device)
        return splits, self._dec_ws[key]

    def _run_layers(self, T: int, Tp: int, Bd: int, nt: int, bt_p, cu_p, ctx_p, ts, tq, lens_d, bt_d, cu_all, ctx_all,
                    slots_all) -> None:
        """Rows [0, Tp): prompt portions (tiles ts / tq over cu_p / ctx_p / bt_p); rows [Tp, T): Bd single new
        rows (lens_d / bt_d).  cu_all / ctx_all / slots_all list both kinds for the recurrent scan."""
        cfg, eps = self.mcfg, self.mcfg.norm_eps
        pos, slots = self._pos, self._slots
        for l, (layer, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            m = layer.mixer
            proj = self._view(self.proj, T, lw.proj.shape[0])
            out = self._view(self.mix_out, T, m.out_width)
            ops.linear(self.xb[:T], lw.proj, proj)
            if m.kind == "attention":
                own = m.kv_from is None
                H, G, dk, dv = m.heads, m.kv_heads, m.dim, m.vdim
                ops.attn_prep(proj, lw.proj_bias, lw.q_norm, lw.k_norm, pos, slots, self.k_cache[l] if own else None,
                              self.v_cache[l] if own else None, H, G, dk, dv, eps, m.q_temp_coef, m.q_temp_every)
                gate_col = (H * dk + (G * (dk + dv) if own else 0)) if m.gate else -1
                kc, vc = self.k_cache[l], self.v_cache[l]
                if nt and self.fast_prefill[l]:
                    ops.paged_attn_prefill_ex(proj[:Tp], proj.stride(0), kc, vc, bt_p, cu_p, ctx_p, ts, tq, out[:Tp], H, G, dk,
                                              m.scale, sink=lw.sink, gate=proj[:Tp, gate_col:] if m.gate else None)
                elif nt:
                    ops.attn_sink_prefill(proj[:Tp], gate_col, kc, vc, bt_p, cu_p, ctx_p, ts, tq, lw.sink, out[:Tp],
                                          H, G, dk, dv, m.scale, tile_rows=self.prefill_tile)
                if Bd and self.fast_decode[l]:
                    splits, ws = self._decode_plan(Bd, m)
                    ops.paged_attn_decode(proj[Tp:T], proj.stride(0), kc, vc, bt_d, lens_d, out[Tp:T], H, G, dk, m.scale,
                                          num_splits=splits, workspace=ws, sink=lw.sink,
                                          gate=proj[Tp:T, gate_col:] if m.gate else None)
                elif Bd:
                    ops.attn_sink_decode(proj[Tp:T], gate_col, kc, vc, bt_d, lens_d, lw.sink, out[Tp:T], H, G, dk, dv,
                                         m.scale)
                self.stats["kernel_launches"] += 2 + (1 if nt else 0) + (1 if Bd else 0)
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
            self._post(T, lw.norm1)
            self.stats["kernel_launches"] += 2
            if layer.mlp is not None:
                act = self._view(self.act, T, layer.mlp.ff)
                ops.linear(self.xb[:T], lw.up, act, relu2=True)        # squared ReLU in the GEMM's epilogue
                ops.linear(act, lw.down, self.y[:T])
                self._post(T, lw.norm2)
                self.stats["kernel_launches"] += 3

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
        ops.sum_layer_norm(None, self.resid32, self.w.final_norm, 1.0, cfg.norm_eps, xb_out=self.x_last[:n], rows=rows,
                           out_scale=cfg.logit_scale)
        lg = self.logits[:n]
        ops.linear(self.x_last[:n], self.w.lm_head, lg)
        ops.sample(lg, temps, seeds, out_idx=self.out_ids[:n])
        self.stats["kernel_launches"] += 3


def runner_class(mcfg):
    """The runner of a model config's family."""
    return LayerListRunner if getattr(mcfg, "family", "") == "layer_list" else ModelRunner
