"""Plain, slow restatement of the Vodavik decoder -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

One function per mechanism, written from the design's equations in torch on the CPU, in one
floating-point type (float64 by default).  It shares nothing with gpustack_b200/: no kernels, no
cache, no scheduler; a sequence is processed whole, token after token where the design recurs.

The design: a post-norm residual stack (x <- LN(a x + f(x)), bias-free layer norm) whose mixers are
either softmax attention without rotation (per-head RMS norm of queries and keys, a query
temperature that grows with the logarithm of the position, a learned per-head sink in the softmax
denominator, a sigmoid output gate, optional reuse of an earlier layer's keys and values) or a
stabilised matrix-memory recurrence (mLSTM), with a relu^2 feed-forward after some mixers.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm_nobias(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) for each position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sink: torch.Tensor, scale: float,
                           q_pos0: int = 0) -> torch.Tensor:
    """q [Tq, H, dk], k [Tk, G, dk], v [Tk, G, dv], sink [H]; query row i sits at position q_pos0 + i
    and sees keys 0 .. q_pos0 + i.  The sink adds exp(sink_h) to the denominator only."""
    Tq, H, _ = q.shape
    Tk, G, dv = v.shape
    rep = H // G
    out = torch.zeros(Tq, H, dv, dtype=q.dtype)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale                                  # [Tq, Tk]
        qi = torch.arange(Tq).unsqueeze(1) + q_pos0
        kj = torch.arange(Tk).unsqueeze(0)
        s = s.masked_fill(kj > qi, float("-inf"))
        m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[h].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True) + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_qkv(h: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict, eps: float, positions: torch.Tensor,
                  with_kv: bool = True):
    """Projections, per-head RMS norms and the query temperature of one attention mixer.
    Returns (q [T,H,dk] already multiplied by its temperature, k [T,G,dk] | None, v [T,G,dv] | None)."""
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, dk)
    q = unit_rms(q, eps) * w["q.norm"]
    qt = spec.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"]).to(q.dtype).reshape(T, 1, 1)
    if not with_kv:
        return q, None, None
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, dk)
    k = unit_rms(k, eps) * w["k.norm"]
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, dv)
    return q, k, v


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict, eps: float, shared_kv=None):
    """Whole-sequence attention mixer; returns (output [T, width], (k, v) as a later layer may reuse them)."""
    T = h.shape[0]
    pos = torch.arange(T)
    q, k, v = attention_qkv(h, w, spec, eps, pos, with_kv=shared_kv is None)
    if shared_kv is not None:
        k, v = shared_kv
    o = sink_softmax_attention(q, k, v, w["sink"], spec["scale"])
    o = o.reshape(T, -1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T, (k, v)


def mlstm_gates(h: torch.Tensor, w: Dict[str, torch.Tensor], cap: float):
    """(log input gate, log forget gate), each [T, heads]."""
    i = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    return i, f


def mlstm_scan(q, k, v, ig, fg, state=None):
    """Token-by-token matrix-memory recurrence.  q, k [T, H, dk]; v [T, H, dv]; ig, fg [T, H].
    state = (S [H, dk, dv], n [H, dk], m [H]) or None for the start (all zero, m = 0).
    Returns (o [T, H, dv], state)."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    if state is None:
        S = torch.zeros(H, dk, dv, dtype=q.dtype)
        n = torch.zeros(H, dk, dtype=q.dtype)
        m = torch.zeros(H, dtype=q.dtype)
    else:
        S, n, m = (t.clone() for t in state)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out, (S, n, m)


def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict, eps: float, state=None):
    H, dk, dv = spec["heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    ig, fg = mlstm_gates(h, w, spec["gate_cap"])
    o, state = mlstm_scan(q, k, v, ig, fg, state)
    o = unit_rms(o, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T, state


def relu2_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.relu(h @ w["up"].T) ** 2 @ w["down"].T


def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    kv: Dict[int, tuple] = {}
    trail = []
    for l, layer in enumerate(cfg["layers"]):
        p = f"l{l}."
        mw = _sub(W, p + "mix.")
        spec = layer["mixer"]
        if layer["type"] == "attention":
            src = spec.get("kv_from")
            y, kv[l] = attention_mixer(x, mw, spec, eps, shared_kv=None if src is None else kv[src])
        elif layer["type"] == "mlstm":
            y, _ = mlstm_mixer(x, mw, spec, eps)
        else:
            raise ValueError(layer["type"])
        x = layer_norm_nobias(alpha * x + y, W[p + "norm1"], eps)
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            x = layer_norm_nobias(alpha * x + relu2_mlp(x, _sub(W, p + "mlp.")), W[p + "norm2"], eps)
        trail.append(x)
    x = layer_norm_nobias(x, W["final.norm"], eps)
    logits = x @ W["head"].T * cfg["logit_scale"]
    return (logits, torch.stack(trail)) if return_layers else logits


def random_weights(cfg: dict, seed: int = 0, std: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with the design's tensor names, scaled so that every mechanism matters:
    sinks, gate biases and norm weights are spread instead of sitting at 0 / 1."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def rnd(*shape, s):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def lin(o, i):
        return rnd(o, i, s=std if std is not None else 1.0 / math.sqrt(i))

    def nw(n):
        return (1.0 + torch.randn(n, generator=g) * 0.2).to(torch.bfloat16)

    w = {"embed": rnd(cfg["vocab"], D, s=1.0), "final.norm": nw(D), "head": lin(cfg["vocab"], D)}
    for l, layer in enumerate(cfg["layers"]):
        p, s = f"l{l}.", layer["mixer"]
        w[p + "norm1"] = nw(D)
        if layer["type"] == "attention":
            H, G, dk, dv = s["heads"], s["kv_heads"], s["dim"], s["vdim"]
            w[p + "mix.q"], w[p + "mix.q.b"], w[p + "mix.q.norm"] = lin(H * dk, D), rnd(H * dk, s=0.3), nw(dk)
            if s.get("kv_from") is None:
                w[p + "mix.k"], w[p + "mix.k.b"], w[p + "mix.k.norm"] = lin(G * dk, D), rnd(G * dk, s=0.3), nw(dk)
                w[p + "mix.v"], w[p + "mix.v.b"] = lin(G * dv, D), rnd(G * dv, s=0.3)
            w[p + "mix.sink"] = rnd(H, s=1.5)
            w[p + "mix.g"], w[p + "mix.o"] = lin(H * dv, D), lin(D, H * dv)
        else:
            H, dk, dv = s["heads"], s["dim"], s["vdim"]
            for n, rows in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv)):
                w[p + "mix." + n] = lin(rows, D)
            w[p + "mix.o"], w[p + "mix.norm"] = lin(D, H * dv), nw(H * dv)
            w[p + "mix.i"], w[p + "mix.i.b"] = lin(H, D), rnd(H, s=1.0)
            w[p + "mix.f"], w[p + "mix.f.b"] = lin(H, D), (3.0 + torch.randn(H, generator=g)).to(torch.bfloat16)
        if layer.get("mlp"):
            w[p + "norm2"] = nw(D)
            w[p + "mlp.up"], w[p + "mlp.down"] = lin(layer["mlp"]["ff"], D), lin(D, layer["mlp"]["ff"])
    return w
