"""Host-side parts of Danipel in the layer-list family: config.json reader, weight fusion, the rotation
frequencies, the library subset a process serving such a model builds, the memory estimate, replay bookkeeping,
and self-consistency of the oracle."""
import json
import math

import pytest
import torch

from gpustack_b200.config import LayerListConfig, ModelConfig, RotarySpec
from gpustack_b200.scheduler import Request, SamplingParams, Scheduler
from gpustack_b200.weights import (layer_list_tensor_shapes, load_layer_list, load_layer_list_dir, random_layer_list_state,
                                   save_layer_list_checkpoint)
from oracle import danipel_oracle as O

F64 = torch.float64


def _cfg():
    rot = {"base": 50.0, "dims": 4, "scaling": {"factor": 4.0, "original": 24, "fast": 8.0, "slow": 1.0}}
    a = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 20, "scale": 0.25, "rot": rot}
    b = {"heads": 5, "dim": 6, "rot_dim": 10, "vdim": 4, "kv_rank": 12, "scale": 0.3, "rot": {"base": 300.0, "dims": 10}, "q_rank": 22}
    moe = {"kind": "moe", "expert": {"ff": 18, "limit": 1.5}, "router": {"experts": 5, "identity": 2, "scale": 1.7, "top": 3},
           "shared": {"ff": 26, "limit": 0.9}}
    return {"architecture": "Danipel", "vocab": 131, "width": 52, "streams": 3, "residual_mult": 0.6, "embedding": {"scale": 2.5},
            "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": a, "mlp": moe},
                       {"type": "latent_attention_2", "mixer": b, "mlp": None},
                       {"type": "latent_attention_2", "mixer": b, "mlp": {"kind": "dense", "ff": 44}}]}


def test_config_reader_round_trip_and_rejections(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    assert c.to_dict() == d and LayerListConfig.from_dict(c.to_dict()).to_dict() == d
    assert c.residual == "streams" and c.norm == "tanh" and c.n_streams == 3 and not c.has_state
    m0, m1 = c.layers[0].mixer, c.layers[1].mixer
    assert (m0.kind, m0.sink, m0.q_rank, m0.rot.layout, m0.rot.yarn_factor) == ("latent_attention", True, 0, "interleaved", 4.0)
    assert (m1.sink, m1.q_rank, m1.rot.layout, m1.rot.yarn_factor) == (False, 22, "half", 0.0)
    assert m0.cache_width == 26 and m0.proj_rows == 3 * 16 + 26 and m1.proj_rows == 22 + 22
    assert c.kv_bytes_per_token() == 2 * (26 + 22 + 22)                  # one shared row per token and layer, not per head
    e = c.layers[0].mlp.moe
    assert (e.experts, e.identity, e.top, e.scale, e.ff, e.limit, e.shared_ff, e.shared_limit) == (5, 2, 3, 1.7, 18, 1.5, 26, 0.9)
    assert c.layers[2].mlp.act == "gelu_tanh" and c.layers[1].mlp is None
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert isinstance(ModelConfig.from_pretrained(str(tmp_path)), LayerListConfig)
    # defaults: no streams key = one plain residual, multiplier and embedding scale 1, no identity, no shared expert
    p = json.loads(json.dumps(d))
    for k in ("streams", "residual_mult", "embedding"):
        del p[k]
    del p["layers"][0]["mlp"]["shared"], p["layers"][0]["mlp"]["router"]["identity"]
    cp = LayerListConfig.from_dict(p)
    assert (cp.streams, cp.n_streams, cp.residual_mult, cp.embed_scale) == (0, 1, 1.0, 1.0)
    assert cp.layers[0].mlp.moe.identity == 0 and cp.layers[0].mlp.moe.shared_ff == 0
    for where, bad in (("type", "conv"), ("mlp", {"kind": "sparse", "ff": 8})):
        x = json.loads(json.dumps(d))
        x["layers"][1][where] = bad
        with pytest.raises(ValueError):
            LayerListConfig.from_dict(x)
    x = json.loads(json.dumps(d))
    x["layers"][0]["mixer"]["rot"]["dims"] = 8                           # wider than the rotated part
    with pytest.raises(ValueError):
        LayerListConfig.from_dict(x)
    x = json.loads(json.dumps(d))
    x["layers"][0]["mlp"]["router"]["top"] = 8                           # more than there are router outputs
    with pytest.raises(ValueError):
        LayerListConfig.from_dict(x)


def test_rotation_frequencies_with_and_without_scaling():
    for rot in ({"base": 50.0, "dims": 4, "scaling": {"factor": 4.0, "original": 24, "fast": 8.0, "slow": 1.0}},
                {"base": 1e6, "dims": 32, "scaling": {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}},
                {"base": 250000.0, "dims": 16}):
        sc = rot.get("scaling") or {}
        f, mag = RotarySpec(dims=rot["dims"], base=rot["base"], yarn_factor=sc.get("factor", 0.0), yarn_original=sc.get("original", 0.0),
                            yarn_fast=sc.get("fast", 0.0), yarn_slow=sc.get("slow", 0.0)).frequencies()
        fo, mo = O.rotary_frequencies(rot)
        assert torch.allclose(torch.tensor(f, dtype=F64), fo, rtol=1e-13) and abs(mag - mo) < 1e-14
    f, mag = RotarySpec(dims=32, base=1e6, yarn_factor=8.0, yarn_original=512, yarn_fast=32.0, yarn_slow=1.0).frequencies()
    plain = [1e6 ** (-2.0 * i / 32) for i in range(16)]
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 8.0) < 1e-18 and plain[5] / 8 < f[5] < plain[5]   # fast pairs kept, slow ones divided
    assert abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-15


def test_weight_fusion_layout_and_checkpoint_round_trip(tmp_path):
    d = _cfg()
    c = LayerListConfig.from_dict(d)
    sd = O.random_weights(d, seed=3)
    assert {k: tuple(v.shape) for k, v in sd.items()} == layer_list_tensor_shapes(c) == O.tensor_shapes(d)
    assert "l1.hc2.in" not in sd and "l1.norm2" not in sd and "l1.mix.sink" not in sd and "l0.mix.sink" in sd
    w = load_layer_list(c, lambda k: sd[k], "cpu")
    a, b = w.layers[0], w.layers[1]
    assert torch.equal(a.proj, torch.cat([sd["l0.mix.q"], sd["l0.mix.dkv"]])) and a.uq is None
    assert torch.equal(b.proj, torch.cat([sd["l1.mix.dq"], sd["l1.mix.dkv"]])) and torch.equal(b.uq, sd["l1.mix.uq"])
    assert a.sink.dtype == torch.float32 and b.sink is None
    for h in range(3):                                                   # per head, W_uk transposed for the query absorption
        assert torch.equal(a.uk_t[h], sd["l0.mix.uk"][h * 10:(h + 1) * 10].T)
    assert a.rot_freq.dtype == F64 and a.rot_freq.shape == (2,) and a.rot_mag > 1.0 and b.rot_mag == 1.0
    hc = a.hc1
    assert hc.dtype == torch.float32 and torch.equal(hc[:3], sd["l0.hc1.in"].float()) and torch.equal(hc[3:6], sd["l0.hc1.out"].float()) \
        and torch.equal(hc[6:].view(3, 3), sd["l0.hc1.mix"].float())
    assert a.norm1_alpha.shape == (1,) and torch.equal(a.norm1_b, sd["l0.norm1.b"])
    assert torch.equal(a.w13[0::2][:18], sd["l0.mlp.e0.gate"]) and torch.equal(a.w13[1::2][18:36], sd["l0.mlp.e1.up"])
    assert torch.equal(a.w2[52:104], sd["l0.mlp.e1.down"]) and a.router.shape == (128, 52) and torch.equal(a.router[:7], sd["l0.mlp.router"]) and not bool(a.router[7:].any()) and a.correction.dtype == torch.float32
    assert torch.equal(a.shared13[0::2], sd["l0.mlp.shared.gate"]) and torch.equal(a.shared2, sd["l0.mlp.shared.down"])
    g = w.layers[2]
    assert torch.equal(g.gate_up[0::2], sd["l2.mlp.gate"]) and torch.equal(g.gate_up[1::2], sd["l2.mlp.up"]) and g.up is None
    assert w.final_norm_alpha.shape == (1,) and b.hc2 is None and b.norm2 is None
    save_layer_list_checkpoint(c, sd, str(tmp_path))
    w2 = load_layer_list_dir(ModelConfig.from_pretrained(str(tmp_path)), str(tmp_path), "cpu")
    assert torch.equal(w2.layers[0].w13, a.w13) and torch.equal(w2.lm_head, w.lm_head)
    bad = dict(sd)
    bad["l0.mix.dkv"] = sd["l0.mix.dkv"][:-1]
    with pytest.raises(ValueError):
        load_layer_list(c, lambda k: bad[k], "cpu")
    # a model without hyper-connections loads as one stream that is read, kept and added to
    p = json.loads(json.dumps(d))
    del p["streams"]
    sp = O.random_weights(p, seed=1)
    assert not any(".hc" in k for k in sp)
    wp = load_layer_list(LayerListConfig.from_dict(p), lambda k: sp[k], "cpu")
    assert torch.equal(wp.layers[0].hc1, torch.ones(3)) and torch.equal(wp.layers[0].hc2, torch.ones(3))
    # the product's own random checkpoints have the same names and shapes
    assert {k: tuple(v.shape) for k, v in random_layer_list_state(c, seed=1).items()} == layer_list_tensor_shapes(c)


def test_library_subset_of_a_streams_model():
    import ctypes

    from gpustack_b200 import build

    c = LayerListConfig.from_dict(_cfg())
    tag, srcs = build.layer_list_sources(c)
    assert tag == "streams_routed" and {"streams.cu", "latent.cu", "moe_biased.cu", "moe.cu", "gemm_simt_grouped.cu"} <= set(srcs)
    assert "mlstm.cu" not in srcs and "attention_prefill_tc.cu" not in srcs and "allreduce.cu" not in srcs
    d = _cfg()
    d["layers"][0]["mlp"] = None
    tag2, srcs2 = build.layer_list_sources(LayerListConfig.from_dict(d))
    assert tag2 == "streams" and "moe.cu" not in srcs2
    h = ctypes.CDLL(str(build.build(sources=srcs, tag=tag)))
    for n in ("b200_streams_step", "b200_embed_streams", "b200_rms_rows", "b200_latent_prep", "b200_linear_simt_grouped",
              "b200_moe_route_biased", "b200_moe_align", "b200_moe_combine_mixed", "b200_attn_sink_prefill", "b200_attn_sink_decode",
              "b200_linear_simt", "b200_gemm_bf16_ex", "b200_sample_f32", "b200_last_error"):
        assert hasattr(h, n), n
    assert not hasattr(h, "b200_mlstm_scan")


def test_vram_estimate_covers_latent_and_routed_layers():
    from gpustack_b200.config import EngineConfig
    from gpustack_b200.resource_fit import estimate

    c = LayerListConfig.from_dict(_cfg())
    e16 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256))
    e32 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256, dtype="float32"))
    assert e16.weights == c.weight_bytes() and e16.kv_bytes_per_token == c.kv_bytes_per_token()
    assert e32.kv_bytes_per_token == 2 * e16.kv_bytes_per_token and e32.workspace > e16.workspace
    n = sum(v.numel() for k, v in O.random_weights(_cfg(), 0).items()
            if not any(t in k for t in ("norm", "hc", "sink", "correction", "embed")))   # the table is looked up, not streamed
    assert c.weight_bytes() == 2 * n


def test_replay_bookkeeping_without_state_slots():
    s = Scheduler(9, 16, 4, 256, 256, None, False, state_slots=0)
    a, b = (Request(req_id=i, prompt_ids=[], params=SamplingParams(max_tokens=0)) for i in "ab")
    s.replay_admit(a)
    s.replay_admit(b)
    s.replay_extend(a, 40)
    s.replay_extend(b, 17)
    assert len(a.blocks) == 3 and len(b.blocks) == 2 and a.state_slot in (-1, None)
    free = s.pool.num_free
    s.replay_finish(a)
    assert s.pool.num_free == free + 3
    s.replay_finish(b)
    assert s.pool.num_free == s.pool.num_total


def test_oracle_mechanisms_are_consistent():
    """Causality (a later token changes nothing before it), the absorbed form of latent attention equals the expanded
    one, identity experts return the input, a model without streams equals one stream with unit weights."""
    d = _cfg()
    W = O.random_weights(d, seed=2)
    toks = torch.randint(0, d["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(d, W, toks)
    assert torch.allclose(O.forward(d, W, toks[:23]), full[:23], atol=1e-9)
    # absorbed latent attention, by hand, for layer 0
    spec, eps = d["layers"][0]["mixer"], d["norm"]["eps"]
    w = {k[len("l0.mix."):]: v.to(F64) for k, v in W.items() if k.startswith("l0.mix.")}
    h = torch.randn(9, d["width"], dtype=F64, generator=torch.Generator().manual_seed(4))
    want = O.latent_attention_mixer(h, w, spec, "latent_attention", eps)
    H, dn, dr, dv, R = spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"], spec["kv_rank"]
    pos = torch.arange(9)
    q = (h @ w["q"].T).view(9, H, dn + dr)
    kv = h @ w["dkv"].T
    row = torch.cat([O.rms_norm(kv[:, :R], w["dkv.norm"], eps), O.rotate(kv[:, R:], pos, spec["rot"], "interleaved")], -1)
    qa = torch.cat([torch.einsum("thd,hdr->thr", q[..., :dn], w["uk"].view(H, dn, R)), O.rotate(q[..., dn:], pos, spec["rot"], "interleaved")], -1)
    k = row.unsqueeze(1).expand(9, H, R + dr)
    o_lat = O.causal_softmax_attention(qa, k, k[..., :R], spec["scale"], sink=w["sink"])
    got = torch.einsum("thr,hvr->thv", o_lat, w["uv"].view(H, dv, R)).reshape(9, H * dv) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-10)
    # identity experts
    m = {"kind": "moe", "expert": {"ff": 4, "limit": 1.0}, "router": {"experts": 1, "identity": 2, "scale": 1.0, "top": 1}}
    x = torch.randn(5, 8, dtype=F64).abs() + 0.1
    ww = {"router": torch.tensor([[-9.0] * 8, [0.0] * 8, [0.0] * 8], dtype=F64), "correction": torch.tensor([0.0, 0.5, 0.0], dtype=F64),
          "e0.gate": torch.randn(4, 8, dtype=F64), "e0.up": torch.randn(4, 8, dtype=F64), "e0.down": torch.randn(8, 4, dtype=F64)}
    ids, wt = O.route(x, ww["router"], ww["correction"], 1, 1.0)
    assert bool((ids == 1).all()) and torch.allclose(wt, torch.ones_like(wt))
    assert torch.allclose(O.moe_mlp(x, ww, m), x)
    # plain residual == one stream with in = out = mix = 1
    p = json.loads(json.dumps(d))
    del p["streams"]
    Wp = {k: v for k, v in W.items() if ".hc" not in k}
    one = dict(p, streams=1)
    W1 = dict(Wp)
    for l, layer in enumerate(p["layers"]):
        for q_ in (1, 2) if layer["mlp"] is not None else (1,):
            W1[f"l{l}.hc{q_}.in"] = W1[f"l{l}.hc{q_}.out"] = torch.ones(1)
            W1[f"l{l}.hc{q_}.mix"] = torch.ones(1, 1)
    assert torch.allclose(O.forward(p, Wp, toks[:12]), O.forward(one, W1, toks[:12]), atol=1e-12)
