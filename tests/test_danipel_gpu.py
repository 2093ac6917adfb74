"""Danipel (layer-list decoder: residual streams, tanh norm, latent attention, gated / routed feed-forward) on the
GPU against the plain restatement in oracle/danipel_oracle.py.

Every test builds its own small configuration and random weights.  Kernel tests compare one mechanism with the
oracle's function; engine tests drive LLMEngine (scheduler pools, runner step functions, CUDA graphs) and compare
logits with the oracle's whole-sequence forward.  float32 must agree to rounding, bfloat16 to bf16 rounding."""
import math

import numpy as np
import pytest
import torch

from oracle import danipel_oracle as O

pytestmark = pytest.mark.gpu

F64 = torch.float64
BF = torch.bfloat16


def _mixer(two, heads, dim, rot_dim, vdim, kv_rank, q_rank=0, dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": dims or rot_dim}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if two:
        m["q_rank"] = q_rank
    return {"type": "latent_attention_2" if two else "latent_attention", "mixer": m}


def _moe(experts, identity, top, ff, limit, scale, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "identity": identity, "scale": scale, "top": top}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def cfg_odd():
    """Nothing is a multiple of 8 or 64: every product takes the CUDA-core path.  Three streams; a rotation that
    covers only part of the rotated width; frequency scaling whose original length (24) the prompts pass; three
    chosen of seven router outputs, two of them identity; a shared expert wider than the routed ones; a layer
    without feed-forward."""
    return {"architecture": "Danipel", "vocab": 131, "width": 52, "streams": 3, "residual_mult": 0.6,
            "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
            "layers": [dict(_mixer(False, 3, 10, 6, 14, 20, dims=4, base=50.0,
                                   scaling={"factor": 4.0, "original": 24, "fast": 8.0, "slow": 1.0}),
                            mlp=_moe(5, 2, 3, 18, 1.5, 1.7, shared=(26, 0.9))),
                       dict(_mixer(True, 5, 6, 10, 4, 12, q_rank=22, base=300.0), mlp=None),
                       dict(_mixer(True, 2, 12, 4, 18, 36, q_rank=10), mlp={"kind": "dense", "ff": 44}),
                       dict(_mixer(False, 4, 4, 8, 10, 28, base=1000.0), mlp=_moe(3, 0, 1, 30, 3.0, 1.0))]}


def cfg_tiles():
    """Widths that the tensor-core GEMMs take in bf16 (multiples of 64), two streams, sixteen heads, routed experts
    without identity or shared expert beside a dense layer, a single head with a wide latent."""
    return {"architecture": "Danipel", "vocab": 256, "width": 128, "streams": 2, "residual_mult": 0.8,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": [dict(_mixer(False, 16, 64, 64, 64, 128, base=1e6,
                                   scaling={"factor": 8.0, "original": 32, "fast": 32.0, "slow": 1.0}),
                            mlp={"kind": "dense", "ff": 192}),
                       dict(_mixer(True, 4, 64, 64, 128, 192, q_rank=64), mlp=_moe(4, 0, 2, 64, 2.0, 2.0)),
                       dict(_mixer(True, 1, 128, 64, 64, 256, q_rank=128), mlp=_moe(6, 2, 2, 128, 1.0, 1.5, shared=(64, 4.0)))]}


def cfg_plain():
    """No hyper-connections (one plain pre-norm residual), residual multiplier and embedding scale 1, one expert of
    which one is chosen, one stream-sized things equal to 1: values a model may happen to make trivial."""
    return {"architecture": "Danipel", "vocab": 77, "width": 40, "norm": {"eps": 1e-6},
            "layers": [dict(_mixer(True, 1, 8, 8, 8, 8, q_rank=8), mlp=_moe(1, 1, 1, 16, 0.5, 1.0)),
                       dict(_mixer(False, 2, 16, 2, 16, 16), mlp={"kind": "dense", "ff": 24})]}


def cfg_one_stream():
    d = cfg_plain()
    d["streams"] = 1
    d["residual_mult"] = 1.3
    return d


CFGS = {"odd": cfg_odd, "tiles": cfg_tiles, "plain": cfg_plain, "one_stream": cfg_one_stream}


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


def _close(got, want, dtype):
    """float32: every logit to rounding.  bfloat16: rounding may overturn a router's close call, which moves that
    position's logits by more than rounding does; so at most one position in twenty may be off (a fault of the
    cache or the batch moves most of them), and the typical position must be well inside the tolerance."""
    if dtype == "float32":
        return _rel(got, want) < TOL[dtype]
    want = want.to(torch.float64).numpy() if isinstance(want, torch.Tensor) else np.asarray(want, dtype=np.float64)
    err = np.abs(np.asarray(got, dtype=np.float64) - want).max(axis=1) / np.abs(want).max()
    return float(np.mean(err > TOL[dtype])) <= 0.05 and float(np.median(err)) < TOL[dtype] / 2


# ------------------------------------------------------------------------------------ mechanisms, one at a time
@pytest.mark.parametrize("S,D", [(1, 37), (2, 64), (3, 52), (4, 200)])
@pytest.mark.parametrize("ydt", [torch.float32, BF])
def test_streams_write_read_and_tanh_norm(S, D, ydt):
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(S * 100 + D)
    T = 7
    X = torch.randn(T, S, D, generator=g) * 2
    y = (torch.randn(T, D, generator=g)).to(ydt)
    hc_w = torch.randn(2 * S + S * S, generator=g)
    hc_r = torch.randn(S, generator=g)
    alpha, w, b = torch.tensor([0.37]), (1 + 0.3 * torch.randn(D, generator=g)).to(BF), (0.2 * torch.randn(D, generator=g)).to(BF)
    Xs = X.permute(1, 0, 2).to(F64)
    newX = O.streams_write(Xs, y.to(F64), hc_w[2 * S:].view(S, S).to(F64), hc_w[S:2 * S].to(F64), 0.7)
    want = O.tanh_norm(O.streams_read(newX, hc_r.to(F64)), alpha.to(F64), w.to(F64), b.to(F64))
    Xd = X.reshape(T, S * D).cuda().contiguous()
    xb = torch.empty(T, D, device="cuda")
    ops.streams_step(Xd, S, y=y.cuda(), hc_write=hc_w.cuda(), mult=0.7, hc_read=hc_r.cuda(), norm=(alpha.cuda(), w.cuda(), b.cuda()), xb_out=xb)
    assert _rel(Xd.view(T, S, D).permute(1, 0, 2), newX) < 2e-6
    assert _rel(xb, want) < 3e-6
    # read only (the step after the embedding), bf16 output
    xb16 = torch.empty(T, D, device="cuda", dtype=BF)
    ops.streams_step(Xd, S, hc_read=hc_r.cuda(), norm=(alpha.cuda(), w.cuda(), b.cuda()), xb_out=xb16)
    assert _rel(xb16.float(), want) < 1e-2
    # write only (the last sublayer), then the final norm of chosen rows over the plain sum of the streams
    X2 = X.reshape(T, S * D).cuda().contiguous()
    ops.streams_step(X2, S, y=y.cuda(), hc_write=hc_w.cuda(), mult=0.7)
    assert _rel(X2.view(T, S, D).permute(1, 0, 2), newX) < 2e-6
    rows = torch.tensor([5, 0, 3], dtype=torch.int32)
    want = O.tanh_norm(newX.sum(0)[rows.long()], alpha.to(F64), w.to(F64), b.to(F64))
    xf = torch.empty(3, D, device="cuda")
    ops.streams_step(X2, S, rows=rows.cuda(), norm=(alpha.cuda(), w.cuda(), b.cuda()), xb_out=xf)
    assert _rel(xf, want) < 3e-6


def test_embedding_fills_every_stream_with_the_scaled_row():
    from gpustack_b200 import ops

    table = torch.randn(11, 20).to(BF)
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32)
    X = torch.empty(4, 3 * 20, device="cuda")
    ops.embed_streams(ids.cuda(), table.cuda(), X, 3, 2.5)
    want = (table.float()[ids.long()] * 2.5).unsqueeze(1).expand(4, 3, 20)
    assert torch.equal(X.view(4, 3, 20).cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_rms_rows_of_a_column_slice(dtype):
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(9, 50, generator=g) * 3).to(dtype)
    w = (1 + 0.3 * torch.randn(22, generator=g)).to(BF)
    out = torch.zeros(9, 22, device="cuda", dtype=dtype)
    ops.rms_rows(x.cuda()[:, 5:27], w.cuda(), out, 1e-5)
    want = O.rms_norm(x[:, 5:27].to(F64), w.to(F64), 1e-5)
    assert _rel(out.float(), want) < (2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("half,dims,dr,scaling", [(False, 8, 8, None), (True, 8, 8, None), (False, 4, 6, {"factor": 4.0, "original": 24, "fast": 8.0, "slow": 1.0}),
                                                  (True, 32, 32, {"factor": 8.0, "original": 64, "fast": 32.0, "slow": 1.0})])
def test_latent_prep_norm_rotation_and_cache_rows(dtype, half, dims, dr, scaling):
    """Positions far beyond the scaling's original length, shuffled cache slots, one padding row (slot -1)."""
    from gpustack_b200 import ops
    from gpustack_b200.config import RotarySpec

    g = torch.Generator().manual_seed(dims + dr)
    T, H, dn, R, page = 6, 3, 10, 20, 4
    rot = {"base": 1000.0, "dims": dims}
    if scaling:
        rot["scaling"] = scaling
    sc = scaling or {}
    spec = RotarySpec(dims=dims, base=1000.0, layout="half" if half else "interleaved", yarn_factor=sc.get("factor", 0.0),
                      yarn_original=sc.get("original", 0.0), yarn_fast=sc.get("fast", 0.0), yarn_slow=sc.get("slow", 0.0))
    f, mag = spec.frequencies()
    fo, mago = O.rotary_frequencies(rot)
    assert np.allclose(np.asarray(f), fo.numpy(), rtol=1e-12) and abs(mag - mago) < 1e-12
    proj = torch.randn(T, 7 + R + dr, generator=g).to(dtype)
    q = torch.randn(T, H * (dn + dr), generator=g).to(dtype)
    w = (1 + 0.3 * torch.randn(R, generator=g)).to(BF)
    pos = torch.tensor([0, 1, 23, 24, 4001, 77], dtype=torch.int32)
    slots = torch.tensor([9, 2, 15, -1, 0, 6], dtype=torch.int32)
    cache = torch.full((4, 1, page, R + dr), 7.0, device="cuda", dtype=dtype)
    qa = torch.zeros(T, H * (R + dr), device="cuda", dtype=dtype)
    ops.latent_prep(proj.cuda(), 7, q.cuda(), w.cuda(), pos.cuda(), slots.cuda(), cache, qa, H, dn, dr, R, dims, half,
                    torch.tensor(f, dtype=F64).cuda(), mag, 1e-5)
    layout = "half" if half else "interleaved"
    c = O.rms_norm(proj[:, 7:7 + R].to(F64), w.to(F64), 1e-5)
    kr = O.rotate(proj[:, 7 + R:].to(F64), pos, rot, layout)
    qr = O.rotate(q.view(T, H, dn + dr)[..., dn:].to(F64), pos, rot, layout)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    flat = cache.view(-1, R + dr).float().cpu()
    for t in range(T):
        if slots[t] < 0:
            continue
        assert _rel(flat[slots[t], :R], c[t]) < tol and _rel(flat[slots[t], R:], kr[t]) < tol
    used = set(int(s) for s in slots if s >= 0)
    assert all(bool((flat[i] == 7.0).all()) for i in range(16) if i not in used)          # nothing else was touched
    assert _rel(qa.view(T, H, R + dr)[..., R:].float(), qr) < tol


@pytest.mark.parametrize("xdt,ydt", [(torch.float32, torch.float32), (BF, BF), (BF, torch.float32)])
def test_per_head_and_gated_linears(xdt, ydt):
    from gpustack_b200 import ops
    from gpustack_b200.weights import _interleave_rows

    g = torch.Generator().manual_seed(5)
    T, H, n, k = 70, 3, 9, 13
    x = torch.randn(T, H * (k + 2), generator=g).to(xdt)
    w = (torch.randn(H, n, k, generator=g) / math.sqrt(k)).to(BF)
    out = torch.zeros(T, H * (n + 1), device="cuda", dtype=ydt)
    ops.head_linear(x.cuda(), w.cuda(), out, H, n=n, k=k, x_head=k + 2, out_head=n + 1)
    want = torch.einsum("thk,hnk->thn", x.view(T, H, k + 2)[..., :k].to(F64), w.to(F64))
    tol = 3e-6 if ydt == torch.float32 else 1e-2
    assert _rel(out.view(T, H, n + 1)[..., :n].float(), want) < tol
    K, N = 52, 37
    xx = torch.randn(T, K, generator=g).to(xdt)
    gate, up = [(2.0 * torch.randn(N, K, generator=g) / math.sqrt(K)).to(BF) for _ in range(2)]
    for act, ref in (("gelu_tanh", lambda a, b: O.gelu_tanh(a) * b),
                     ("clamped_swish", lambda a, b: (lambda gg, uu: gg * torch.sigmoid(1.702 * gg) * (uu + 1))(a.clamp(max=0.8), b.clamp(-0.8, 0.8))),
                     ("silu", lambda a, b: a * torch.sigmoid(a) * b)):
        o = torch.empty(T, N, device="cuda", dtype=ydt)
        ops.gated_linear(xx.cuda(), _interleave_rows(gate, up).cuda(), o, act, 0.8)
        want = ref(xx.to(F64) @ gate.to(F64).T, xx.to(F64) @ up.to(F64).T)
        assert _rel(o.float(), want) < tol, act


@pytest.mark.parametrize("E,ident,top", [(5, 2, 3), (70, 3, 4), (1, 0, 1), (3, 5, 8)])
def test_routing_choice_by_corrected_scores_weights_by_scores(E, ident, top):
    from gpustack_b200 import ops

    g = torch.Generator().manual_seed(E)
    T, n = 50, E + ident
    logits = torch.randn(T, n, generator=g) * 2
    corr = torch.randn(n, generator=g) * 0.3                  # large enough to overturn many choices
    ids = torch.empty(T * top, dtype=torch.int32, device="cuda")
    w = torch.empty(T * top, dtype=torch.float32, device="cuda")
    ops.moe_route_biased(logits.cuda(), corr.cuda(), top, 2.5, ids, w, n)
    s = torch.softmax(logits.to(F64), -1)
    want_ids = torch.topk(s + corr.to(F64), top, dim=-1).indices
    plain_ids = torch.topk(s, top, dim=-1).indices
    if top < n:
        assert not torch.equal(want_ids.sort(-1).values, plain_ids.sort(-1).values)      # the correction matters here
    got_ids = ids.view(T, top).cpu().long()
    assert torch.equal(got_ids, want_ids)
    ws = torch.gather(s, 1, want_ids)
    assert _rel(w.view(T, top), ws / (ws.sum(-1, keepdim=True) + 1e-20) * 2.5) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("E,ident,top,ff,shared", [(5, 2, 3, 18, (26, 0.9)), (3, 0, 1, 30, None), (70, 1, 2, 8, None)])
def test_routed_experts_with_identity_and_shared_expert(dtype, E, ident, top, ff, shared):
    from gpustack_b200 import ops
    from gpustack_b200.weights import _interleave_rows

    g = torch.Generator().manual_seed(E + ff)
    T, D = 45, 28
    spec = _moe(E, ident, top, ff, 1.2, 1.7, shared)
    w = {"router": 3 * torch.randn(E + ident, D, generator=g) / math.sqrt(D), "correction": 0.1 * torch.randn(E + ident, generator=g)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = [2 * torch.randn(ff, D, generator=g) / math.sqrt(D) for _ in range(2)]
        w[f"e{e}.down"] = torch.randn(D, ff, generator=g) / math.sqrt(ff)
    if shared:
        w["shared.gate"], w["shared.up"] = [2 * torch.randn(shared[0], D, generator=g) / math.sqrt(D) for _ in range(2)]
        w["shared.down"] = torch.randn(D, shared[0], generator=g) / math.sqrt(shared[0])
    w = {k: v.to(BF) for k, v in w.items()}
    x = torch.randn(T, D, generator=g).to(dtype)
    want = O.moe_mlp(x.to(F64), {k: v.to(F64) for k, v in w.items()}, spec)
    ws = ops.RoutedWorkspace(64, top, E + ident, D, ff, dtype, "cuda")
    w13 = torch.cat([_interleave_rows(w[f"e{e}.gate"], w[f"e{e}.up"]) for e in range(E)]).cuda()
    w2 = torch.cat([w[f"e{e}.down"] for e in range(E)]).cuda()
    sh = None
    xd = x.cuda()
    if shared:
        a = torch.empty(T, shared[0], device="cuda", dtype=dtype)
        ops.gated_linear(xd, _interleave_rows(w["shared.gate"], w["shared.up"]).cuda(), a, "clamped_swish", shared[1])
        sh = torch.empty(T, D, device="cuda")
        ops.linear(a, w["shared.down"].cuda(), sh)
    out = torch.empty(T, D, device="cuda")
    for _ in range(2):          # the workspace is reused as it is
        ops.routed_experts(xd, w["router"].cuda(), w["correction"].float().cuda(), w13, w2, ws, out, E, ident, top, 1.7, ff, 1.2, shared=sh)
    assert _rel(out, want) < (5e-6 if dtype == torch.float32 else 2e-2)


def test_tensor_core_routes_of_the_per_head_gated_and_routed_products():
    """bf16 shapes that the tcgen05 GEMMs take (K multiples of 64, 16-byte aligned slices): per-head products over strided
    views, the gated epilogues, the grouped expert GEMMs with an fp32 weighted output; 300 rows = several tiles."""
    from gpustack_b200 import ops
    from gpustack_b200.weights import _interleave_rows

    g = torch.Generator().manual_seed(9)
    T, H, n, k = 300, 3, 40, 64
    x = torch.randn(T, H * (k + 8), generator=g).to(BF)
    w = (torch.randn(H, n, k, generator=g) / math.sqrt(k)).to(BF)
    out = torch.zeros(T, H * (n + 8), device="cuda", dtype=BF)
    ops.head_linear(x.cuda(), w.cuda(), out, H, n=n, k=k, x_head=k + 8, out_head=n + 8)
    want = torch.einsum("thk,hnk->thn", x.view(T, H, k + 8)[..., :k].to(F64), w.to(F64))
    assert _rel(out.view(T, H, n + 8)[..., :n].float(), want) < 1e-2
    assert bool((out.view(T, H, n + 8)[..., n:] == 0).all())                 # the gaps between the heads' outputs stay untouched
    K, N = 128, 192
    xx = torch.randn(T, K, generator=g).to(BF)
    gate, up = [(2.0 * torch.randn(N, K, generator=g) / math.sqrt(K)).to(BF) for _ in range(2)]
    for act, lim, ref in (("gelu_tanh", 0.0, lambda a, b: O.gelu_tanh(a) * b),
                          ("clamped_swish", 0.7, lambda a, b: (lambda gg, uu: gg * torch.sigmoid(1.702 * gg) * (uu + 1))(a.clamp(max=0.7), b.clamp(-0.7, 0.7)))):
        o = torch.empty(T, N, device="cuda", dtype=BF)
        ops.gated_linear(xx.cuda(), _interleave_rows(gate, up).cuda(), o, act, lim)
        assert _rel(o.float(), ref(xx.to(F64) @ gate.to(F64).T, xx.to(F64) @ up.to(F64).T)) < 1e-2, act
    E, ident, top, ff, D = 4, 1, 2, 128, 256
    spec = _moe(E, ident, top, ff, 1.2, 1.7)
    wm = {"router": 3 * torch.randn(E + ident, D, generator=g) / math.sqrt(D), "correction": 0.1 * torch.randn(E + ident, generator=g)}
    for e in range(E):
        wm[f"e{e}.gate"], wm[f"e{e}.up"] = [2 * torch.randn(ff, D, generator=g) / math.sqrt(D) for _ in range(2)]
        wm[f"e{e}.down"] = torch.randn(D, ff, generator=g) / math.sqrt(ff)
    wm = {k_: v.to(BF) for k_, v in wm.items()}
    xm = torch.randn(T, D, generator=g).to(BF)
    want = O.moe_mlp(xm.to(F64), {k_: v.to(F64) for k_, v in wm.items()}, spec)
    ws = ops.RoutedWorkspace(320, top, E + ident, D, ff, BF, "cuda")
    w13 = torch.cat([_interleave_rows(wm[f"e{e}.gate"], wm[f"e{e}.up"]) for e in range(E)]).cuda()
    w2 = torch.cat([wm[f"e{e}.down"] for e in range(E)]).cuda()
    outm = torch.empty(T, D, device="cuda")
    for rows in (T, 3):                                                      # prompt-sized and decode-sized steps
        ops.routed_experts(xm[:rows].cuda().contiguous(), wm["router"].cuda(), wm["correction"].float().cuda(), w13, w2, ws, outm[:rows], E, ident, top,
                           1.7, ff, 1.2)
        assert ws.xp is not None                                            # the tensor-core path ran
        assert _rel(outm[:rows], want[:rows]) < 2e-2


def _latent_case(dtype, n_keys, page, H, R, dr, seed, perm=True):
    """Cache rows for one sequence of n_keys tokens in shuffled pages, junk in the pages it does not own."""
    g = torch.Generator().manual_seed(seed)
    C = torch.randn(n_keys, R + dr, generator=g).to(dtype)
    nb = (n_keys + page - 1) // page
    order = torch.randperm(nb + 3, generator=g)[:nb] if perm else torch.arange(nb)
    cache = torch.full((nb + 3, 1, page, R + dr), 50.0, dtype=dtype)
    for j in range(n_keys):
        cache[order[j // page], 0, j % page] = C[j]
    return C, cache.cuda(), order.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("H,R,dr,sink", [(3, 20, 6, True), (16, 128, 64, False), (1, 256, 8, True), (20, 512, 64, True),
                                         (3, 64, 16, False), (8, 192, 32, True), (2, 384, 32, False), (2, 192, 16, True),
                                         (32, 128, 32, False), (40, 64, 32, True)])
def test_attention_over_the_latent_cache_prefill_and_decode(dtype, H, R, dr, sink):
    """Absorbed form: every head scores against the same cache rows and takes their first R entries as values.
    A portion of 37 rows after 130 cached tokens (three 64-key blocks, ten pages), then single rows, against the
    expanded-per-head oracle.  bf16 shapes with R a multiple of 64 run on the tensor-core kernel, the rest on the
    generic one."""
    from gpustack_b200 import ops

    page, ctx, new = 16, 130, 37
    n = ctx + new
    C, cache, order = _latent_case(dtype, n, page, H, R, dr, seed=H + R)
    g = torch.Generator().manual_seed(1)
    q = torch.randn(new, H, R + dr, generator=g).to(dtype)
    sk = (torch.randn(H, generator=g) * 1.5) if sink else None
    scale = 1.2 / math.sqrt(R + dr)
    k = C.to(F64).unsqueeze(1).expand(n, H, R + dr)
    want = O.causal_softmax_attention(q.to(F64), k, k[..., :R], scale, sink=None if sk is None else sk.to(F64), q_pos0=ctx)
    bt = torch.zeros(1, 16, dtype=torch.int32)
    bt[0, :len(order)] = order
    tile = ops.attn_sink_prefill_tile()
    ts, tq = ops.build_prefill_tiles([new], tile, [ctx])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")   # noqa: E731
    out = torch.zeros(new, H * R, device="cuda", dtype=dtype)
    qd = q.reshape(new, -1).cuda()
    skd = None if sk is None else sk.cuda()
    ops.latent_attn_prefill(qd, cache, bt.cuda(), i32([0, new]), i32([ctx]), i32(ts), i32(tq), skd, out, H, R, dr, scale)
    tol = 5e-6 if dtype == torch.float32 else 1.5e-2
    assert _rel(out.view(new, H, R).float(), want) < tol
    rows = [0, 1, 17, new - 1]
    o4 = torch.zeros(len(rows) + 1, H * R, device="cuda", dtype=dtype)          # the last row: a padding row without keys
    bt4 = bt.repeat(len(rows) + 1, 1).cuda()
    ops.latent_attn_decode(qd[rows + [0]].contiguous(), cache, bt4, i32([ctx + r + 1 for r in rows] + [0]), skd, o4, H, R, dr, scale)
    assert _rel(o4[:len(rows)].view(len(rows), H, R).float(), want[rows]) < tol
    assert bool(torch.isfinite(o4[-1].float()).all())
    if dtype == BF and ops.latent_attn_covers(H, R, dr):       # the keys cut into ranges (some of them empty) and merged
        for ns in (2, 3, 16):
            ws = ops.latent_attn_decode_workspace(len(rows) + 1, H, R, 16, "cuda")
            ws.fill_(float("nan"))
            o5 = torch.zeros_like(o4)
            ops.latent_attn_decode(qd[rows + [0]].contiguous(), cache, bt4, i32([ctx + r + 1 for r in rows] + [0]), skd, o5, H, R, dr, scale,
                                   num_splits=ns, workspace=ws)
            assert _rel(o5[:len(rows)].view(len(rows), H, R).float(), want[rows]) < tol, ns
            assert bool((o5[-1] == 0).all())


@pytest.mark.parametrize("kernel", ["prefill", "decode"])
@pytest.mark.parametrize("far", [0, 15, 16, 17, 63, 64, 250])
@pytest.mark.parametrize("dtype,H,R,dr", [(torch.float32, 4, 24, 8), (BF, 4, 64, 16), (BF, 16, 128, 32)])
def test_one_far_key_stands_out_and_the_next_token_stays_invisible(kernel, far, dtype, H, R, dr):
    """400 cached tokens; the key at `far` (first token, page and key-block borders, far back) is made to dominate every
    head's scores, so the output must be its latent.  A still larger key one place AFTER the query must not be seen."""
    from gpustack_b200 import ops

    page, n = 16, 400
    g = torch.Generator().manual_seed(far)
    C = torch.randn(n + 1, R + dr, generator=g) * 0.1
    q = torch.randn(1, H, R + dr, generator=g) * 0.1
    direction = torch.zeros(R + dr)
    direction[R + 1] = 1.0
    C[far] += 40 * direction
    C[n] += 90 * direction                       # position n: the future for a query at n - 1
    q = q + direction
    C, q = C.to(dtype), q.to(dtype)
    nb = (n + 1 + page - 1) // page
    cache = torch.zeros(nb, 1, page, R + dr, dtype=dtype)
    cache.view(-1, R + dr)[:n + 1] = C
    cache = cache.cuda()
    bt = torch.arange(nb, dtype=torch.int32).view(1, -1).cuda()
    out = torch.zeros(1, H * R, device="cuda", dtype=dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")   # noqa: E731
    sink = torch.zeros(H, device="cuda")
    if kernel == "prefill":
        ts, tq = ops.build_prefill_tiles([1], ops.attn_sink_prefill_tile(), [n - 1])
        ops.latent_attn_prefill(q.reshape(1, -1).cuda(), cache, bt, i32([0, 1]), i32([n - 1]), i32(ts), i32(tq), sink, out, H, R, dr, 1.0)
    else:
        ops.latent_attn_decode(q.reshape(1, -1).cuda(), cache, bt, i32([n]), sink, out, H, R, dr, 1.0)
    for h in range(H):
        assert torch.allclose(out.view(H, R)[h].float().cpu(), C[far, :R].float(), atol=1e-4 if dtype == torch.float32 else 2e-3), (kernel, far, h)


# ------------------------------------------------------------------------------------ whole models
@pytest.fixture(scope="module", params=list(CFGS))
def model(request):
    cfg = CFGS[request.param]()
    return cfg, O.random_weights(cfg, seed=3 + len(request.param))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer(model, dtype):
    cfg, W = model
    toks = _tokens(cfg, 70, 1)
    trail = []
    want = O.forward(cfg, W, toks, layer_outputs=trail)
    eng = _engine(cfg, W, dtype)
    run = eng.runner
    seen, join = [], run._join

    def spy(T, l, q):
        join(T, l, q)
        if q == 2 or cfg["layers"][l]["mlp"] is None:
            seen.append(run.resid32[:T].view(T, run.S, -1).sum(1).cpu().clone())

    run._join = spy
    got = eng.replay_step([("a", toks, list(range(len(toks))))], ["a"])
    run._join = join
    assert len(seen) == len(cfg["layers"])
    for l in range(len(seen)):
        assert _rel(seen[l], trail[l]) < TOL[dtype] * 2, f"residual stream after layer {l}"
    assert _close(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_and_single_tokens_match_the_whole_prompt(model, dtype):
    """One prompt, token by token, and portions of changing size down to two tokens (page size 16: cuts inside and at
    page borders): the logits at a position do not depend on the cut (float32: to rounding)."""
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
def test_mixed_batches_of_unequal_requests_with_reused_pages(model, dtype):
    """Five requests of unequal length through four sequence slots and too few pages for all of them at once: portions
    of some ride beside single tokens of others, a finished request's pages go to the next one.  Every request's
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
    assert eng.runner.stats.get("mixed_steps", 0) >= 4 and eng.runner.stats["decode_steps"] >= 1


def test_long_decoding_past_the_scaling_length_in_float32():
    """300 single-token steps after a short prompt through the captured decode graphs: the positions pass the
    frequency scaling's original length many times over and the decode kernel walks 20 pages."""
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
    """LLMEngine.generate: continuous batching of six prompts over four sequence slots, chunked prefill (token
    budget 48), decode steps.  The oracle is teacher-forced on the engine's tokens; wherever its top-2 margin is
    decisive the engine's token is its argmax."""
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
