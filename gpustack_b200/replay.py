"""Replay of a recorded schedule: given token ids go through the engine step by step and the logits of chosen
rows are written out.  Nothing is sampled.

Steps arrive on standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

`entries` are one batch (prompt portions beside single decoded tokens); a request is admitted at its first entry
and may skip steps; the requests in `end` give their KV blocks and state slot back after the step.  For a step in
which something is wanted, OUT/<step>.f32 receives the logits [wanted rows, vocab] as little-endian fp32, entries
in order; after every step a line `done <step>` is printed.

The engine is the serving engine (LLMEngine.replay_step -> the runner's prefill / mixed / decode step functions,
the scheduler's block pool and state-slot pool); its KV pool holds --max-tokens tokens (each request rounded up
to whole 16-token pages) and it has --max-seqs sequence and state slots, so pages and slots are reused.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np


def run(model: str, dtype: str, out_dir: str, max_tokens: int, max_seqs: int = 4, stdin=None, stdout=None) -> int:
    stdin = sys.stdin if stdin is None else stdin
    stdout = sys.stdout if stdout is None else stdout
    from . import build, lib
    from .config import EngineConfig, ModelConfig

    if dtype not in ("bfloat16", "float32"):
        print(f"unknown dtype {dtype}", file=sys.stderr)
        return 2
    mcfg = ModelConfig.from_pretrained(model)
    family = getattr(mcfg, "family", "llama")
    if dtype == "float32" and family != "layer_list":
        print("this model family has no 32-bit path", file=sys.stderr)
        return 3
    if family == "layer_list":
        lib.prefer_subset(*build.layer_list_sources(mcfg))     # a fresh checkout compiles what this model launches, no more
    import torch

    from .engine import LLMEngine

    if not torch.cuda.is_available():
        print("no CUDA device visible: this engine has no CPU path", file=sys.stderr)
        return 2
    torch.backends.cuda.matmul.allow_tf32 = False
    block = 16
    pages = (max_tokens + block - 1) // block
    ecfg = EngineConfig(model=model, dtype=dtype, max_model_len=max(block, max_tokens), max_num_seqs=max_seqs,
                        max_num_batched_tokens=max(max_tokens, max_seqs), num_gpu_blocks=pages + 1, block_size=block,
                        enable_prefix_caching=False, max_logit_rows=max(max_tokens, max_seqs))
    eng = LLMEngine.from_engine_config(ecfg)
    os.makedirs(out_dir, exist_ok=True)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want") or []) for e in msg.get("entries", [])]
        if entries:
            logits = eng.replay_step(entries, msg.get("end") or [])
        else:
            logits = np.zeros((0, mcfg.vocab_size), dtype=np.float32)
            for rid in msg.get("end") or []:
                r = eng.requests.pop(rid, None)
                if r is not None:
                    eng.sched.replay_finish(r)
        if logits.shape[0]:
            tmp = os.path.join(out_dir, f".{msg['step']}.part")
            with open(tmp, "wb") as f:
                f.write(np.ascontiguousarray(logits[:, :mcfg.vocab_size], dtype="<f4").tobytes())
            os.replace(tmp, os.path.join(out_dir, f"{msg['step']}.f32"))
        stdout.write(f"done {msg['step']}\n")
        stdout.flush()
    eng.shutdown()
    return 0
