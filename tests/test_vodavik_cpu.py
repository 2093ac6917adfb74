"""Host-side parts of the layer-list decoder family (Vodavik): config.json reader, weight fusion, state-slot
pool, scheduler admission with state slots, the replay bookkeeping, and self-consistency of the oracle."""
import json

import numpy as np
import pytest
import torch

from gpustack_b200.config import LayerListConfig, ModelConfig, architecture_of
from gpustack_b200.kv_cache import StateSlotPool
from gpustack_b200.scheduler import Request, SamplingParams, Scheduler
from gpustack_b200.weights import (layer_list_tensor_shapes, load_layer_list, random_layer_list_state,
                                   save_layer_list_checkpoint)
from oracle import vodavik_oracle as O


def _cfg():
    a = {"heads": 6, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.25, "q_temp": {"coef": 0.7, "every": 3}}
    return {"architecture": "Vodavik", "vocab": 101, "width": 52, "postln_alpha": 1.7, "logit_scale": 0.8, "norm": {"eps": 1e-5},
            "layers": [{"type": "mlstm", "mixer": {"heads": 2, "dim": 10, "vdim": 36, "gate_cap": 9.0}, "mlp": {"kind": "dense", "ff": 44}},
                       {"type": "attention", "mixer": a, "mlp": None},
                       {"type": "attention", "mixer": dict(a, kv_from=1), "mlp": {"kind": "dense", "ff": 60}}]}


def test_config_reader_round_trip_and_registry(tmp_path):
    d = _cfg()
    assert architecture_of(d) == "Vodavik" and architecture_of({"architectures": ["Qwen2ForCausalLM"]}) == "Qwen2ForCausalLM"
    c = LayerListConfig.from_dict(d)
    assert c.to_dict() == d
    assert c.has_state and c.kv_owner(0) is None and c.kv_owner(1) == 1 and c.kv_owner(2) == 1
    assert c.kv_bytes_per_token() == 3 * (20 + 12) * 2          # only the layer that owns its pages
    assert c.state_bytes_per_seq() == 4 * 2 * (10 * 36 + 2 * 10 + 2)
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert isinstance(ModelConfig.from_pretrained(str(tmp_path)), LayerListConfig)     # the class is chosen by config.json
    for bad in ({"type": "conv"}, {"mixer": dict(d["layers"][2]["mixer"], kv_from=0)}, {"mixer": dict(d["layers"][2]["mixer"], kv_from=2)},
                {"mlp": {"kind": "moe", "ff": 8}}):
        e = json.loads(json.dumps(d))
        e["layers"][2].update(bad)
        with pytest.raises(ValueError):
            LayerListConfig.from_dict(e)


def test_weight_fusion_layout_and_checkpoint_round_trip(tmp_path):
    c = LayerListConfig.from_dict(_cfg())
    sd = random_layer_list_state(c, seed=3)
    assert {k: tuple(v.shape) for k, v in sd.items()} == layer_list_tensor_shapes(c)
    assert "l2.mix.k" not in sd and "l2.mix.k.norm" not in sd and "l2.mix.q.b" in sd      # a kv_from layer has queries only
    w = load_layer_list(c, lambda k: sd[k], "cpu")
    a = w.layers[1]
    assert torch.equal(a.proj, torch.cat([sd["l1.mix.q"], sd["l1.mix.k"], sd["l1.mix.v"], sd["l1.mix.g"]]))
    assert torch.equal(a.proj_bias, torch.cat([sd["l1.mix.q.b"], sd["l1.mix.k.b"], sd["l1.mix.v.b"]]))
    assert a.sink.dtype == torch.float32 and a.norm2 is None
    b = w.layers[2]
    assert torch.equal(b.proj, torch.cat([sd["l2.mix.q"], sd["l2.mix.g"]])) and b.k_norm is None and b.up is not None
    r = w.layers[0]
    assert torch.equal(r.gates, torch.cat([sd["l0.mix.i"], sd["l0.mix.f"]])) and r.gate_bias.shape == (4,)
    save_layer_list_checkpoint(c, sd, str(tmp_path))
    from gpustack_b200.weights import load_layer_list_dir

    w2 = load_layer_list_dir(ModelConfig.from_pretrained(str(tmp_path)), str(tmp_path), "cpu")
    assert torch.equal(w2.layers[2].proj, b.proj) and torch.equal(w2.lm_head, w.lm_head)
    bad = dict(sd)
    bad["l1.mix.q"] = sd["l1.mix.q"][:-1]
    with pytest.raises(ValueError):
        load_layer_list(c, lambda k: bad[k], "cpu")


def test_state_slot_pool_reuses_the_last_freed_slot():
    p = StateSlotPool(3)
    a, b, c = p.allocate(), p.allocate(), p.allocate()
    assert sorted((a, b, c)) == [0, 1, 2] and p.num_free == 0
    with pytest.raises(MemoryError):
        p.allocate()
    p.free(b)
    assert p.allocate() == b
    with pytest.raises(ValueError):
        p.free(b) or p.free(b)


def test_scheduler_admits_only_with_a_free_state_slot_and_gives_it_back():
    s = Scheduler(num_blocks=64, block_size=16, max_num_seqs=8, max_num_batched_tokens=64, max_model_len=128, eos_token_id=None,
                  enable_prefix_caching=True, state_slots=2)
    assert not s.pool.caching                        # recurrent state: no prefix reuse
    reqs = [Request(req_id=f"r{i}", prompt_ids=[1, 2, 3, 4 + i], params=SamplingParams(max_tokens=2, ignore_eos=True)) for i in range(3)]
    for r in reqs:
        s.add(r)
    plan = s.schedule()
    assert [r.req_id for r in plan.reqs] == ["r0", "r1"] and sorted(r.state_slot for r in plan.reqs) == [0, 1]
    assert reqs[2].state_slot == -1 and s.slots.num_free == 0
    s.update_prefill(plan, [7, 8])
    assert list(s.state_slot[:2]) == [reqs[0].state_slot, reqs[1].state_slot]
    plan = s.schedule()                              # r2 still waits: decode only
    assert plan.batch == 2
    s.update_decode(plan, np.asarray([5, 6], dtype=np.int32))      # both reach max_tokens: slots and blocks come back
    assert s.slots.num_free == 2 and reqs[0].state_slot == -1
    plan = s.schedule()
    assert [r.req_id for r in plan.reqs] == ["r2"] and reqs[2].state_slot in (0, 1)
    s.abort("r2")
    assert s.slots.num_free == 2 and s.pool.num_free == s.pool.num_total


def test_replay_bookkeeping_takes_and_returns_pages_and_slots():
    s = Scheduler(num_blocks=6, block_size=16, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=80, eos_token_id=None,
                  state_slots=2)
    a = Request(req_id="a", prompt_ids=[], params=SamplingParams(max_tokens=0))
    s.replay_admit(a)
    s.replay_extend(a, 17)
    assert len(a.blocks) == 2 and a.state_slot >= 0
    a.num_computed = 17
    s.replay_extend(a, 15)
    assert len(a.blocks) == 2
    s.replay_extend(a, 16)
    assert len(a.blocks) == 3
    b = Request(req_id="b", prompt_ids=[], params=SamplingParams(max_tokens=0))
    s.replay_admit(b)
    with pytest.raises(MemoryError):
        s.replay_extend(b, 60)                       # 4 pages wanted, 2 left
    with pytest.raises(MemoryError):
        s.replay_admit(Request(req_id="c", prompt_ids=[], params=SamplingParams(max_tokens=0)))
    s.replay_finish(a)
    s.replay_extend(b, 60)
    s.replay_finish(b)
    assert s.pool.num_free == s.pool.num_total and s.slots.num_free == 2 and not s.prefilling


def test_oracle_recurrence_and_attention_do_not_depend_on_the_cut():
    """The oracle's own mechanisms: a scan in portions equals the whole scan; attention rows of a prefix equal the
    prefix's own rows (causality); the sink only shrinks the weights."""
    g = torch.Generator().manual_seed(0)
    T, H, dk, dv = 40, 2, 6, 5
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for d in (dk, dk, dv))
    ig, fg = torch.randn(T, H, generator=g, dtype=torch.float64), -torch.rand(T, H, generator=g, dtype=torch.float64)
    whole, _ = O.mlstm_scan(q, k, v, ig, fg)
    st, parts = None, []
    for lo, hi in ((0, 1), (1, 3), (3, 20), (20, 40)):
        o, st = O.mlstm_scan(q[lo:hi], k[lo:hi], v[lo:hi], ig[lo:hi], fg[lo:hi], st)
        parts.append(o)
    assert torch.allclose(torch.cat(parts), whole, atol=1e-12)
    sink = torch.tensor([0.5, -2.0], dtype=torch.float64)
    full = O.sink_softmax_attention(q, k, v, sink, 0.4)
    assert torch.allclose(O.sink_softmax_attention(q[:13], k[:13], v[:13], sink, 0.4), full[:13], atol=1e-12)
    tail = O.sink_softmax_attention(q[13:], k, v, sink, 0.4, q_pos0=13)
    assert torch.allclose(tail, full[13:], atol=1e-12)
    none = O.sink_softmax_attention(q, k, v, torch.full((2,), -1e30, dtype=torch.float64), 0.4)
    assert torch.allclose(none[0], v[0], atol=1e-12) and not torch.allclose(full[0], v[0])
    t = O.query_temperature(torch.tensor([0, 1, 2, 3, 5, 8]), 0.5, 3)
    assert torch.allclose(t, 1 + 0.5 * torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0, 3.0, 4.0], dtype=torch.float64)))


def test_family_libraries_link_alone_and_export_what_the_runner_calls():
    """A process that serves one layer-list model builds a library from that family's sources only; both variants
    (generic attention only / plus the tensor-core attention kernels) must link without the rest and export every
    entry point the runner can reach for such a model."""
    import ctypes

    from gpustack_b200 import build

    generic = LayerListConfig.from_dict(_cfg())
    tag, srcs = build.layer_list_sources(generic)
    assert tag == "layer_list" and "attention.cu" not in srcs and "moe.cu" not in srcs
    d = _cfg()
    d["layers"][1]["mixer"].update(dim=64, vdim=64)
    d["layers"][2]["mixer"].update(dim=64, vdim=64)
    tag_tc, srcs_tc = build.layer_list_sources(LayerListConfig.from_dict(d))
    assert tag_tc == "layer_list_tc" and set(build.ATTENTION_TC_SOURCES) <= set(srcs_tc)
    base = ["b200_linear_simt", "b200_gemm_bf16_ex", "b200_gemm_bf16_relu2", "b200_sum_layer_norm", "b200_embed_rows_f32",
            "b200_relu2", "b200_attn_prep", "b200_attn_sink_prefill", "b200_attn_sink_decode", "b200_mlstm_scan",
            "b200_mlstm_out", "b200_sample_f32", "b200_last_error"]
    for t, s_, names in ((tag, srcs, base), (tag_tc, srcs_tc, base + ["b200_paged_attn_prefill_ex", "b200_paged_attn_decode_ex",
                                                                      "b200_attn_prefill_tile", "b200_attn_decode_splits",
                                                                      "b200_attn_decode_workspace_bytes"])):
        h = ctypes.CDLL(str(build.build(sources=s_, tag=t)))
        for n in names:
            assert hasattr(h, n), (t, n)
    assert not hasattr(ctypes.CDLL(str(build.subset_lib(tag))), "b200_moe_route")


def test_vram_estimate_covers_layer_list_models(tmp_path):
    from gpustack_b200.config import EngineConfig
    from gpustack_b200.resource_fit import estimate

    c = LayerListConfig.from_dict(_cfg())
    e16 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256))
    e32 = estimate(c, EngineConfig(max_model_len=256, max_num_seqs=4, max_num_batched_tokens=256, dtype="float32"))
    assert e16.weights == c.weight_bytes() and e16.kv_bytes_per_token == c.kv_bytes_per_token()
    assert e32.kv_bytes_per_token == 2 * e16.kv_bytes_per_token and e32.workspace > e16.workspace
    assert e16.workspace >= 4 * c.state_bytes_per_seq()
