"""Vodavik (layer-list decoder) on the GPU against the plain restatement in oracle/vodavik_oracle.py.

Every test builds its own small configuration and random weights.  Kernel tests compare one mechanism with the
oracle's function of the same name; engine tests drive LLMEngine (scheduler pools, runner step functions, CUDA
graphs) and compare logits with the oracle's whole-sequence forward.  In float32 the engine must agree to
rounding (the tolerances are a few 1e-5 of the logit scale); in bfloat16 to bf16 rounding."""
import math

import numpy as np
import pytest
import torch

from oracle import vodavik_oracle as O

pytestmark = pytest.mark.gpu

F64 = torch.float64


def _attn(heads, kv_heads, dim, vdim, every=0, coef=0.0, kv_from=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def cfg_odd():
    """Nothing is a multiple of 8: every projection takes the CUDA-core path; a recurrent layer comes first; the
    query temperature changes every 3 positions; the third attention layer reads the first one's pages."""
    a = _attn(6, 3, 20, 12, every=3, coef=0.7)
    return {"architecture": "Vodavik", "vocab": 101, "width": 52, "postln_alpha": 1.7, "logit_scale": 0.8,
            "norm": {"eps": 1e-5},
            "layers": [{"type": "mlstm", "mixer": {"heads": 2, "dim": 10, "vdim": 36, "gate_cap": 9.0}, "mlp": {"kind": "dense", "ff": 44}},
                       {"type": "attention", "mixer": a, "mlp": None},
                       {"type": "attention", "mixer": _attn(2, 2, 8, 40), "mlp": {"kind": "dense", "ff": 28}},
                       {"type": "attention", "mixer": dict(a, kv_from=1), "mlp": {"kind": "dense", "ff": 60}},
                       {"type": "mlstm", "mixer": {"heads": 3, "dim": 44, "vdim": 8, "gate_cap": 15.0}, "mlp": None}]}


def cfg_tiles():
    """Tensor-core friendly widths (multiples of 64): the projections run on the tcgen05 GEMM in bf16; equal key /
    value widths, one kv head per query head in one layer, a single recurrent head, temperature every position."""
    return {"architecture": "Vodavik", "vocab": 256, "width": 128, "postln_alpha": 3.0, "logit_scale": 1.0,
            "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": _attn(4, 4, 32, 32, every=1, coef=0.25), "mlp": {"kind": "dense", "ff": 192}},
                       {"type": "mlstm", "mixer": {"heads": 1, "dim": 64, "vdim": 64, "gate_cap": 12.0}, "mlp": None},
                       {"type": "attention", "mixer": _attn(8, 2, 16, 32, kv_from=None), "mlp": None},
                       {"type": "mlstm", "mixer": {"heads": 4, "dim": 16, "vdim": 48, "gate_cap": 20.0}, "mlp": {"kind": "dense", "ff": 64}}]}


def cfg_tc():
    """Equal key / value widths of a tensor-core tile: in bf16 the first attention layer (128 wide, groups of 4) runs on the
    tcgen05 prefill kernel and the split-KV decode kernel with sink and gate; the second (groups of 8: another tile size)
    and the third (64 wide) keep the generic prefill kernel, with 32-row tiles cut in two, and the fast decode kernel."""
    return {"architecture": "Vodavik", "vocab": 320, "width": 256, "postln_alpha": 2.0, "logit_scale": 0.7,
            "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": _attn(8, 2, 128, 128, every=16, coef=0.3), "mlp": {"kind": "dense", "ff": 256}},
                       {"type": "mlstm", "mixer": {"heads": 2, "dim": 64, "vdim": 96, "gate_cap": 10.0}, "mlp": None},
                       {"type": "attention", "mixer": _attn(8, 1, 128, 128), "mlp": None},
                       {"type": "attention", "mixer": _attn(4, 2, 64, 64, every=7, coef=0.5), "mlp": {"kind": "dense", "ff": 128}},
                       {"type": "attention", "mixer": _attn(8, 2, 128, 128, kv_from=0), "mlp": None}]}


def _engine(cfg, weights, dtype, blocks=64, seqs=4, mbt=256, eager=False):
    from gpustack_b200.config import EngineConfig, LayerListConfig
    from gpustack_b200.engine import LLMEngine

    ecfg = EngineConfig(dtype=dtype, max_model_len=512, max_num_seqs=seqs, max_num_batched_tokens=mbt, num_gpu_blocks=blocks,
                        enable_prefix_caching=False, max_logit_rows=mbt, enforce_eager=eager)
    return LLMEngine.from_engine_config(ecfg, mcfg=LayerListConfig.from_dict(cfg), state_dict={k: v.cuda() for k, v in weights.items()})


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _rel(got, want):
    want = want.to(torch.float64).numpy() if isinstance(want, torch.Tensor) else want
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(1e-9, np.abs(want).max()))


TOL = {"float32": 3e-5, "bfloat16": 4e-2}


# ------------------------------------------------------------------------------------ mechanisms, one at a time
@pytest.mark.parametrize("D", [37, 200, 1024])
@pytest.mark.parametrize("ydt", [torch.float32, torch.bfloat16])
def test_sum_layer_norm(D, ydt):
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(D)
    x = torch.randn(9, D, generator=g) * 3 + 1.5
    y = (torch.randn(9, D, generator=g) * 2).to(ydt)
    w = (1 + 0.3 * torch.randn(D, generator=g)).to(torch.bfloat16)
    want = O.layer_norm_nobias(2.5 * x.to(F64) + y.to(F64), w.to(F64), 1e-5)
    xo = torch.empty(9, D, device="cuda")
    xb = torch.empty(9, D, device="cuda", dtype=torch.bfloat16)
    ops.sum_layer_norm(y.cuda(), x.cuda(), w.cuda(), 2.5, 1e-5, x_out=xo, xb_out=xb)
    assert _rel(xo.cpu(), want) < 2e-6
    assert _rel(xb.float().cpu(), want) < 1e-2
    # gather form (no branch output), with an output scale
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    want = O.layer_norm_nobias(x.to(F64)[rows.long()], w.to(F64), 1e-5) * 0.5
    xf = torch.empty(3, D, device="cuda")
    ops.sum_layer_norm(None, x.cuda(), w.cuda(), 1.0, 1e-5, xb_out=xf, rows=rows.cuda(), out_scale=0.5)
    assert _rel(xf.cpu(), want) < 2e-6


@pytest.mark.parametrize("M,N,K", [(1, 4, 33), (5, 7, 320), (70, 130, 52), (3, 64, 128)])
@pytest.mark.parametrize("xdt,ydt", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16)])
def test_linear_any_shape(M, N, K, xdt, ydt):
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(xdt)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    b = torch.randn(N, generator=g).to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=ydt)
    ops.linear(x.cuda(), w.cuda(), out)
    want = x.to(F64) @ w.to(F64).T
    assert _rel(out.float().cpu(), want) < (2e-6 if ydt == torch.float32 else 1e-2)
    ops.linear(x.cuda(), w.cuda(), out, bias=b.cuda())
    assert _rel(out.float().cpu(), want + b.to(F64)) < (2e-6 if ydt == torch.float32 else 1e-2)


def test_relu2_and_embedding():
    from gpustack_b200 import ops

    u = torch.randn(5, 33)
    for dt in (torch.float32, torch.bfloat16):
        got = ops.relu2(u.to(dt).cuda().clone())
        assert _rel(got.float().cpu(), torch.relu(u.to(dt).to(F64)) ** 2) < (1e-6 if dt == torch.float32 else 1e-2)
    table = torch.randn(11, 20).to(torch.bfloat16)
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32)
    x32 = torch.empty(4, 20, device="cuda")
    xb = torch.empty(4, 20, device="cuda", dtype=torch.bfloat16)
    ops.embed_rows(ids.cuda(), table.cuda(), x32, xb)
    assert torch.equal(x32.cpu(), table[ids.long()].float()) and torch.equal(xb.cpu(), table[ids.long()])


def _paged(k, v, page, dtype, perm_seed=0, extra_blocks=3):
    """Scatter [T, G, d] keys / values into shuffled pages; returns (k_cache, v_cache, block_table row)."""
    T, G, dk = k.shape
    dv = v.shape[-1]
    nb = (T + page - 1) // page
    perm = torch.randperm(nb + extra_blocks, generator=torch.Generator().manual_seed(perm_seed))[:nb] + 1
    kc = torch.full((nb + extra_blocks + 1, G, page, dk), 7.0)
    vc = torch.full((nb + extra_blocks + 1, G, page, dv), -7.0)       # junk everywhere a key must not be read
    for t in range(T):
        kc[perm[t // page], :, t % page] = k[t]
        vc[perm[t // page], :, t % page] = v[t]
    return kc.to(dtype).cuda(), vc.to(dtype).cuda(), perm.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv", [(6, 3, 20, 12), (4, 4, 32, 32), (8, 1, 72, 136)])
def test_attention_prep_prefill_decode(dtype, H, G, dk, dv):
    """bias + head norms + temperature + page scatter, then prompt portions and single rows over shuffled pages:
    a portion that starts in the middle of a page with earlier context, sinks of both signs."""
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(H * dk + dv)
    D, T, page, eps = 40, 83, 16, 1e-5
    spec = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 0.3, "q_temp": {"coef": 0.6, "every": 5}}
    w = {"q": torch.randn(H * dk, D, generator=g) / 6, "k": torch.randn(G * dk, D, generator=g) / 6,
         "v": torch.randn(G * dv, D, generator=g) / 6, "q.b": torch.randn(H * dk, generator=g) * 0.3,
         "k.b": torch.randn(G * dk, generator=g) * 0.3, "v.b": torch.randn(G * dv, generator=g) * 0.3,
         "q.norm": 1 + 0.2 * torch.randn(dk, generator=g), "k.norm": 1 + 0.2 * torch.randn(dk, generator=g),
         "sink": torch.randn(H, generator=g) * 2}
    w = {k_: v_.to(torch.bfloat16) for k_, v_ in w.items()}
    h = torch.randn(T, D, generator=g).to(torch.bfloat16)
    gate = torch.randn(T, H * dv, generator=g).to(dtype)
    w64 = {k_: v_.to(F64) for k_, v_ in w.items()}
    q, k, v = O.attention_qkv(h.to(F64), w64, spec, eps, torch.arange(T))
    want = O.sink_softmax_attention(q, k, v, w64["sink"], spec["scale"]).reshape(T, -1) * torch.sigmoid(gate.to(F64))
    # product path: raw projections (no bias) -> prep -> attention
    raw = torch.cat([h.to(F64) @ w64["q"].T, h.to(F64) @ w64["k"].T, h.to(F64) @ w64["v"].T, gate.to(F64)], dim=1).to(dtype).cuda()
    bias = torch.cat([w["q.b"], w["k.b"], w["v.b"]]).cuda()
    nb = (T + page - 1) // page
    perm = (torch.randperm(nb + 2, generator=g)[:nb] + 1).to(torch.int32)
    kc = torch.full((nb + 3, G, page, dk), 9.0, dtype=dtype, device="cuda")
    vc = torch.full((nb + 3, G, page, dv), -9.0, dtype=dtype, device="cuda")
    pos = torch.arange(T, dtype=torch.int32)
    slots = (perm[(pos // page).long()] * page + pos % page).to(torch.int32)
    ops.attn_prep(raw, bias, w["q.norm"].cuda(), w["k.norm"].cuda(), pos.cuda(), slots.cuda(), kc, vc, H, G, dk, dv, eps, 0.6, 5)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert _rel(raw[:, :H * dk].float().cpu(), q.reshape(T, -1)) < tol
    out = torch.zeros(T, H * dv, dtype=dtype, device="cuda")
    gate_col = H * dk + G * (dk + dv)
    bt = torch.zeros(2, nb + 4, dtype=torch.int32)
    bt[0, :nb] = perm
    bt[1, :nb] = perm
    # one sequence as two portions in ONE launch is not allowed (same rows), so: rows [0, 27) then [27, T)
    for lo, hi in ((0, 27), (27, T)):
        tile = ops.attn_sink_prefill_tile()
        ts, tq = ops.build_prefill_tiles([hi - lo], tile, [lo])
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")   # noqa: E731
        ops.attn_sink_prefill(raw[lo:hi], gate_col, kc, vc, bt.cuda(), i32([0, hi - lo]), i32([lo]), i32(ts), i32(tq),
                              w["sink"].float().cuda(), out[lo:hi], H, G, dk, dv, spec["scale"])
    assert _rel(out.float().cpu(), want) < tol
    # single rows: positions at and around page borders, the first token, the last
    rows = [0, 1, 15, 16, 17, 31, 32, 48, T - 1]
    outd = torch.zeros(len(rows), H * dv, dtype=dtype, device="cuda")
    btd = bt[:1].repeat(len(rows), 1).cuda()
    ops.attn_sink_decode(raw[rows], gate_col, kc, vc, btd, torch.tensor([r + 1 for r in rows], dtype=torch.int32, device="cuda"),
                         w["sink"].float().cuda(), outd, H, G, dk, dv, spec["scale"])
    assert _rel(outd.float().cpu(), want[rows]) < tol
    # without a sink and without a gate the denominators differ: both branches exist
    outn = torch.zeros(len(rows), H * dv, dtype=dtype, device="cuda")
    ops.attn_sink_decode(raw[rows], -1, kc, vc, btd, torch.tensor([r + 1 for r in rows], dtype=torch.int32, device="cuda"),
                         None, outn, H, G, dk, dv, spec["scale"])
    plain = O.sink_softmax_attention(q, k, v, torch.full((H,), -1e30, dtype=F64), spec["scale"]).reshape(T, -1)
    assert _rel(outn.float().cpu(), plain[rows]) < tol


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
def test_attention_finds_one_far_key_and_respects_the_causal_edge(kernel):
    """One key among hundreds is made to stand out (its dot product with the query is far larger than the others): the
    output must be that key's value -- at a page border, many pages back -- and a key ONE position after the
    query must not be seen however large its score."""
    from gpustack_b200 import ops

    H = G = 1
    dk, dv, page, T = 24, 8, 16, 400
    g = torch.Generator().manual_seed(5)
    for far in (0, 15, 16, 17, 255, 256, 383):
        k = torch.randn(T, 1, dk, generator=g) * 0.05
        v = torch.randn(T, 1, dv, generator=g)
        qpos = 390
        q = torch.randn(dk, generator=g) * 0.05
        k[far, 0] = 0
        k[far, 0, 3] = 40.0
        k[qpos + 1, 0, 3] = 80.0          # the future key: would win if it were visible
        q[3] = 1.0
        kc, vc, perm = _paged(k, v, page, torch.float32, perm_seed=far)
        bt = torch.zeros(1, 40, dtype=torch.int32)
        bt[0, :len(perm)] = perm
        proj = torch.zeros(qpos + 1, dk) if kernel == "prefill" else torch.zeros(1, dk)
        proj[-1] = q
        out = torch.zeros(proj.shape[0], dv, device="cuda")
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")   # noqa: E731
        sink = torch.tensor([-3.0], device="cuda")
        if kernel == "prefill":
            # a portion [380, 391) on top of 380 cached tokens
            lo = 380
            ts, tq = ops.build_prefill_tiles([qpos + 1 - lo], ops.attn_sink_prefill_tile(), [lo])
            ops.attn_sink_prefill(proj[lo:].cuda(), -1, kc, vc, bt.cuda(), i32([0, qpos + 1 - lo]), i32([lo]), i32(ts), i32(tq),
                                  sink, out[lo:], H, G, dk, dv, 1.0)
        else:
            ops.attn_sink_decode(proj.cuda(), -1, kc, vc, bt.cuda(), i32([qpos + 1]), sink, out, H, G, dk, dv, 1.0)
        assert torch.allclose(out[-1].cpu(), v[far, 0], atol=1e-4), (kernel, far)


@pytest.mark.parametrize("form", ["serial", "chunk"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(2, 10, 36), (1, 64, 64), (3, 44, 8), (2, 200, 40)])
def test_mlstm_scan_portions_and_slots(dtype, H, dk, dv, form):
    """The recurrence over portions of 1, 2 and many tokens with the state carried in a slot; a slot that held
    another sequence is reused; two sequences in one launch."""
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(dk * dv + H)
    T, cap = 75, 6.0
    mk = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc)   # noqa: E731
    q, k, v = mk(T, H, dk).to(dtype), mk(T, H, dk).to(dtype), mk(T, H, dv).to(dtype)
    gi, gf = mk(T, H, sc=3.0), mk(T, H, sc=3.0) + 2.0
    bias = mk(2 * H).to(torch.bfloat16)
    ig = cap * torch.tanh((gi.to(F64) + bias[:H].to(F64)) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((gf.to(F64) + bias[H:].to(F64)) / cap))
    want, _ = O.mlstm_scan(q.to(F64) * dk ** -0.5, k.to(F64), v.to(F64), ig, fg)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).cuda()
    gates = torch.cat([gi, gf], dim=1).float().cuda().contiguous()
    slots = 3
    Z = ops.mlstm_state_slices(dv)
    S = torch.full((slots, H, dv, dk), 5.0, device="cuda")          # junk: a fresh sequence must not read it
    n = torch.full((slots, H, Z, dk), -5.0, device="cuda")
    m = torch.full((slots, H, Z), 11.0, device="cuda")
    o = torch.zeros(T, H * dv, device="cuda")
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")   # noqa: E731
    cuts = [0, 1, 3, 5, 22, 23, 40, T]
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        ops.mlstm_scan(proj[lo:hi], 0, H * dk, 2 * H * dk, gates[lo:hi], bias.cuda(), i32([0, hi - lo]), i32([lo]), i32([1]),
                       S, n, m, o[lo:hi], H, dk, dv, cap, max_len=(hi - lo) if form == "chunk" else 1)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    assert _rel(o.cpu(), want.reshape(T, -1)) < tol
    assert float(S[0].min()) == 5.0 and float(S[2].max()) == 5.0       # other slots untouched
    # the same slot again from position 0, beside a second sequence that continues in slot 2 (skipped: slot -1)
    o2 = torch.zeros(T, H * dv, device="cuda")
    ops.mlstm_scan(proj, 0, H * dk, 2 * H * dk, gates, bias.cuda(), i32([0, 30, T]), i32([0, 30]), i32([1, -1]), S, n, m, o2,
                   H, dk, dv, cap, max_len=T if form == "chunk" else 1)
    assert _rel(o2[:30].cpu(), want.reshape(T, -1)[:30]) < tol
    assert float(o2[30:].abs().max()) == 0.0


def test_mlstm_out_norm_gate():
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(3)
    T, H, dv = 7, 3, 20
    o = torch.randn(T, H * dv, generator=g) * 4
    gate = torch.randn(T, H * dv, generator=g)
    w = (1 + 0.2 * torch.randn(H * dv, generator=g)).to(torch.bfloat16)
    want = O.unit_rms(o.to(F64).reshape(T, H, dv), 1e-5).reshape(T, -1) * w.to(F64) * torch.sigmoid(gate.to(F64))
    out = torch.empty(T, H * dv, device="cuda")
    ops.mlstm_out(o.cuda(), gate.cuda(), 0, w.cuda(), out, H, dv, 1e-5)
    assert _rel(out.cpu(), want) < 2e-6


# ------------------------------------------------------------------------------------ the engine
@pytest.fixture(scope="module", params=["odd", "tiles", "tc"])
def model(request):
    cfg = {"odd": cfg_odd, "tiles": cfg_tiles, "tc": cfg_tc}[request.param]()
    return cfg, O.random_weights(cfg, seed={"odd": 11, "tiles": 12, "tc": 13}[request.param])


def test_tensor_core_attention_is_chosen_where_the_shapes_allow():
    cfg = cfg_tc()
    r = _engine(cfg, O.random_weights(cfg, seed=1), "bfloat16").runner
    assert r.prefill_tile == 32 and r.fast_prefill == {0: True, 2: False, 3: False, 4: True}
    assert all(r.fast_decode.values())
    r = _engine(cfg, O.random_weights(cfg, seed=1), "float32").runner
    assert not any(r.fast_prefill.values()) and not any(r.fast_decode.values()) and r.prefill_tile == 16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer(model, dtype):
    cfg, W = model
    toks = _tokens(cfg, 70, 1)
    want, trail = O.forward(cfg, W, toks, return_layers=True)
    eng = _engine(cfg, W, dtype)
    run = eng.runner
    seen, post = [], run._post

    def spy(T, w):
        post(T, w)
        seen.append(run.resid32[:T].cpu().clone())

    run._post = spy
    got = eng.replay_step([("a", toks, list(range(len(toks))))], ["a"])
    run._post = post
    k = 0
    for l, layer in enumerate(cfg["layers"]):
        k += 1 + (layer["mlp"] is not None)
        assert _rel(seen[k - 1], trail[l]) < TOL[dtype] * 2, f"residual stream after layer {l}"
    assert _rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_single_tokens_match_the_whole_prompt(model, dtype):
    """The same tokens as one prompt, token by token, and in portions of changing size down to two tokens: the
    logits at a position do not depend on the cut (float32: to rounding)."""
    cfg, W = model
    toks = _tokens(cfg, 90, 2)
    want = O.forward(cfg, W, toks)
    eng = _engine(cfg, W, dtype)
    whole = eng.replay_step([("w", toks, list(range(len(toks))))], ["w"])
    one = np.concatenate([eng.replay_step([("t", toks[i:i + 1], [0])], ["t"] if i == len(toks) - 1 else []) for i in range(len(toks))])
    parts, pos, i = [], 0, 0
    sizes = [2, 3, 16, 2, 17, 1, 5, 31, 2]
    while pos < len(toks):
        c = min(sizes[i % len(sizes)], len(toks) - pos)
        parts.append(eng.replay_step([("p", toks[pos:pos + c], list(range(c)))], ["p"] if pos + c == len(toks) else []))
        pos, i = pos + c, i + 1
    parts = np.concatenate(parts)
    for got in (whole, one, parts):
        assert _rel(got, want) < TOL[dtype]
    if dtype == "float32":
        assert _rel(one, whole) < 1e-5 and _rel(parts, whole) < 1e-5
    assert eng.sched.pool.num_free == eng.sched.pool.num_total and eng.sched.slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests_with_reused_pages_and_slots(model, dtype):
    """Five requests of unequal length through a pool of four state slots and too few pages for all of them at once: portions
    of some ride beside single tokens of others, a finished request's pages and slot go to the next one.  Every
    request's logits equal those of the request alone."""
    cfg, W = model
    lens = [61, 9, 120, 33, 47]
    reqs = {f"r{i}": _tokens(cfg, n, 20 + i) for i, n in enumerate(lens)}
    want = {k: O.forward(cfg, W, t).numpy() for k, t in reqs.items()}
    eng = _engine(cfg, W, dtype, blocks=17, seqs=4)     # 16 pages: the five requests need 19, so pages are reused
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    # step plans: (request, tokens this step)
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
        assert _rel(np.concatenate(got[k]), want[k]) < TOL[dtype], k
    assert eng.sched.pool.num_free == eng.sched.pool.num_total and eng.sched.slots.num_free == 4
    assert eng.runner.stats.get("mixed_steps", 0) >= 4 and eng.runner.stats["decode_steps"] >= 1


def test_long_decoding_and_temperature_steps_in_float32():
    """300 single-token steps after a short prompt: the recurrent state and the running maximum stay exact, the
    query temperature passes many of its steps, the decode kernel walks 20 pages."""
    cfg = cfg_odd()
    W = O.random_weights(cfg, seed=5)
    toks = _tokens(cfg, 320, 9)
    want = O.forward(cfg, W, toks)
    eng = _engine(cfg, W, "float32")
    out = [eng.replay_step([("a", toks[:20], list(range(20)))], [])]
    for i in range(20, len(toks)):
        out.append(eng.replay_step([("a", toks[i:i + 1], [0])], ["a"] if i == len(toks) - 1 else []))
    assert _rel(np.concatenate(out), want) < TOL["float32"]
    assert eng.runner.stats["graph_replays"] >= 290          # the decode steps ran as captured graphs


@pytest.mark.parametrize("dtype,eager", [("float32", True), ("bfloat16", False)])
def test_greedy_generation_through_the_scheduler(model, dtype, eager):
    """LLMEngine.generate: continuous batching of six prompts over four sequence slots (admission waits for a slot),
    chunked prefill (token budget 48), decode steps.  The oracle is teacher-forced on the engine's tokens; wherever
    its top-2 margin is decisive the engine's token is its argmax."""
    from gpustack_b200.scheduler import SamplingParams

    cfg, W = model
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
    assert eng.sched.slots.num_free == 4 and eng.sched.pool.num_free == eng.sched.pool.num_total


def test_float32_is_refused_by_families_without_a_32_bit_path():
    from gpustack_b200.config import EngineConfig, tiny_llama
    from gpustack_b200.engine import LLMEngine
    from gpustack_b200.lib import B200Error

    with pytest.raises(B200Error):
        LLMEngine.from_engine_config(EngineConfig(dtype="float32", max_num_seqs=2, num_gpu_blocks=16, max_model_len=64),
                                     mcfg=tiny_llama())


def test_seeded_temperature_and_nucleus_sampling_through_the_engine():
    """The family uses the engine's samplers unchanged: in-kernel Gumbel-max for plain temperature sampling (same
    seed = same tokens whatever the batch), host re-sampling for nucleus requests; both differ from greedy."""
    from gpustack_b200.scheduler import SamplingParams

    cfg = cfg_tiles()
    W = O.random_weights(cfg, seed=3)
    prompts = [_tokens(cfg, n, 70 + n) for n in (9, 30, 18)]
    eng = _engine(cfg, W, "bfloat16", seqs=4)
    greedy = eng.generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True))
    hot = SamplingParams(max_tokens=16, ignore_eos=True, temperature=1.5, seed=123)
    a = eng.generate(prompts, hot)
    b = eng.generate(prompts[::-1], hot)[::-1]                       # other batch order, same seeds
    assert a == b and a != greedy
    nuc = SamplingParams(max_tokens=16, ignore_eos=True, temperature=1.5, top_p=0.8, seed=5)
    c, d = eng.generate(prompts[:1], nuc), eng.generate(prompts[:1], nuc)
    assert c == d and all(0 <= t < cfg["vocab"] for t in c[0])
    assert eng.sched.slots.num_free == 4
