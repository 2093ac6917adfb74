"""Side benchmark of the layer-list family (Vodavik) beside the closest Llama-class model of equal layer sizes.

`python bench.py --family vodavik` prints ONE JSON line (not the serving benchmark's line; that workload and its
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
from .config import (AttentionSpec, EngineConfig, LayerListConfig, LayerSpec, MLPSpec, MLSTMSpec, ModelConfig)

ROOT = Path(__file__).resolve().parent.parent
SIZES = {
    # name: width, heads, kv_heads, head width, ff, vocab
    "2k": (2048, 16, 4, 128, 8192, 32000),
    "4k": (4096, 32, 8, 128, 14336, 32000),
}


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


def run(sizes=("2k", "4k"), seqs=4, prompt=2048, batch=64, decode_steps=32, log=None):
    log = log or (lambda m: print(m, file=sys.stderr, flush=True))
    hbm, fl, how = _peaks()
    out = {"bench": "family", "family": "vodavik", "dtype": "bf16", "data": "synthetic", "peaks": how,
           "workload": {"prefill": f"{seqs} x {prompt}", "decode": f"{batch} rows at context {prompt}", "layers": 4}, "sizes": {}}
    for size in sizes:
        log(f"size {size}: {SIZES[size]}")
        o = {"model": {}, "kernels": {}}
        for name, cfg in (("vodavik", vodavik_config(size)), ("llama", llama_config(size))):
            o["model"][name] = _model_numbers(cfg, seqs, prompt, batch, decode_steps, log)
        o["kernels"] = _kernel_numbers(size, seqs * prompt, batch, prompt, log)
        out["sizes"][size] = o
    return out
