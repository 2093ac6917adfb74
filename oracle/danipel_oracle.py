"""Plain, slow restatement of the Danipel decoder -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

One function per mechanism, written from the design's equations in torch on the CPU, in one
floating-point type (float64 by default).  It shares nothing with gpustack_b200/: no kernels, no
cache, no scheduler; a sequence is processed whole and keys / values are expanded per head.

The design: several parallel residual streams joined by learned scalar weights (static
hyper-connections), a tanh norm without statistics, attention whose keys and values are expanded
from one small latent per token plus one rotated key part shared by all heads (two variants: direct
queries / interleaved rotation with optional YaRN frequency scaling / softmax sink, and latent
queries / half-split rotation / plain softmax), and a feed-forward that is either a gated GELU
layer or a routed mixture of clamped gated experts with identity experts and a shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------ norms
def tanh_norm(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """tanh(alpha x) w + b: no mean, no variance."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------ streams
def streams_read(X: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """X [s, T, D] -> sum_s in[s] X[s]."""
    return torch.einsum("s,std->td", w_in, X)


def streams_write(X: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor, m: float) -> torch.Tensor:
    """new X[t] = sum_s mix[s, t] X[s] + m out[t] y  (all streams from the old ones)."""
    return torch.einsum("sr,std->rtd", mix, X) + m * w_out.reshape(-1, 1, 1) * y.unsqueeze(0)


# ------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot: dict, dtype=torch.float64):
    """(frequencies [dims / 2], factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """x [T, ..., w]: the first rot.dims entries of the last axis are rotated, the rest pass.  layout
    'interleaved': pairs (2i, 2i+1); 'half': pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype).reshape(-1, *([1] * (x.dim() - 1))) * f            # [T, ..., dims/2]
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    elif layout == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


# ------------------------------------------------------------------------------ attention
def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                             sink: Optional[torch.Tensor] = None, q_pos0: int = 0) -> torch.Tensor:
    """q [Tq, H, dk], k [Tk, H, dk], v [Tk, H, dv]; query row i is at position q_pos0 + i and sees keys
    0 .. q_pos0 + i.  sink [H]: exp(sink_h) joins the denominator only."""
    Tq, H, _ = q.shape
    Tk = k.shape[0]
    out = torch.zeros(Tq, H, v.shape[-1], dtype=q.dtype)
    qi = torch.arange(Tq).unsqueeze(1) + q_pos0
    kj = torch.arange(Tk).unsqueeze(0)
    for h in range(H):
        s = (q[:, h] @ k[:, h].T) * scale
        s = s.masked_fill(kj > qi, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, h]
    return out


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict, variant: str, eps: float,
                           positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Whole-sequence latent attention.  variant 'latent_attention': q = W_q h, interleaved rotation,
    softmax sink; 'latent_attention_2': q = W_uq rms(W_dq h), half-split rotation, plain softmax."""
    T = h.shape[0]
    H, dn, dr, dv, R = spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"], spec["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    two = variant == "latent_attention_2"
    layout = "half" if two else "interleaved"
    if two:
        q = rms_norm(h @ w["dq"].T, w["dq.norm"], eps) @ w["uq"].T
    else:
        q = h @ w["q"].T
    q = q.reshape(T, H, dn + dr)
    kv = h @ w["dkv"].T                                                        # [T, R + dr]
    c = rms_norm(kv[:, :R], w["dkv.norm"], eps)
    k_rot = rotate(kv[:, R:], pos, spec["rot"], layout)                        # one per token, all heads share it
    q_rot = rotate(q[..., dn:], pos, spec["rot"], layout)
    k_nope = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    qq = torch.cat([q[..., :dn], q_rot], dim=-1)
    kk = torch.cat([k_nope, k_rot.unsqueeze(1).expand(T, H, dr)], dim=-1)
    o = causal_softmax_attention(qq, kk, v, float(spec["scale"]), sink=None if two else w["sink"])
    return o.reshape(T, H * dv) @ w["o"].T


# ------------------------------------------------------------------------------ feed-forward
def dense_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int, scale: float):
    """(chosen expert ids [T, top], their weights [T, top]): softmax over every router output, choice by
    score + correction, weights from the scores alone, normalised over the chosen, times scale."""
    s = torch.softmax(h @ router.T, dim=-1)
    ids = torch.topk(s + correction, top, dim=-1).indices
    wts = torch.gather(s, 1, ids)
    wts = wts / (wts.sum(dim=-1, keepdim=True) + 1e-20) * scale
    return ids, wts


def moe_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], spec: dict) -> torch.Tensor:
    r = spec["router"]
    n_real, n_id = int(r["experts"]), int(r.get("identity", 0) or 0)
    ids, wts = route(h, w["router"], w["correction"], int(r["top"]), float(r.get("scale", 1.0)))
    out = torch.zeros_like(h)
    limit = float(spec["expert"]["limit"])
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            if e >= n_real:                           # identity expert: the input itself
                assert e < n_real + n_id
                out[t] += wts[t, j] * h[t]
            else:
                out[t] += wts[t, j] * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    if spec.get("shared"):
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(spec["shared"]["limit"]))
    return out


# ------------------------------------------------------------------------------ model
def _sub(state: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in state.items() if k.startswith(prefix)}


def forward(cfg: dict, state: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence.  cfg is the config.json dict.  layer_outputs: a list
    that receives the sum of the streams after every layer."""
    st = {k: v.to(dtype) for k, v in state.items()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    S = int(cfg.get("streams", 0) or 0)
    x = st["embed"][torch.tensor(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    X = x.unsqueeze(0).repeat(max(S, 1), 1, 1)

    def norm(u, name):
        return tanh_norm(u, st[name + ".alpha"], st[name], st[name + ".b"])

    for l, layer in enumerate(cfg["layers"]):
        p = f"l{l}."
        subs = [(1, lambda u, layer=layer, p=p: latent_attention_mixer(u, _sub(st, p + "mix.", dtype), layer["mixer"],
                                                                       layer["type"], eps))]
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] == "dense":
                subs.append((2, lambda u, p=p: dense_mlp(u, _sub(st, p + "mlp.", dtype))))
            else:
                subs.append((2, lambda u, layer=layer, p=p: moe_mlp(u, _sub(st, p + "mlp.", dtype), layer["mlp"])))
        for q, fn in subs:
            if S:
                u = streams_read(X, st[p + f"hc{q}.in"])
                y = fn(norm(u, p + f"norm{q}"))
                X = streams_write(X, y, st[p + f"hc{q}.mix"], st[p + f"hc{q}.out"], m)
            else:
                X = X + m * fn(norm(X[0], p + f"norm{q}")).unsqueeze(0)
        if layer_outputs is not None:
            layer_outputs.append(X.sum(dim=0))
    x = X.sum(dim=0)
    return norm(x, "final.norm") @ st["head"].T


# ------------------------------------------------------------------------------ random models for tests
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    D, S = cfg["width"], int(cfg.get("streams", 0) or 0)
    sh: Dict[str, tuple] = {"embed": (cfg["vocab"], D), "head": (cfg["vocab"], D)}

    def norm(name):
        sh[name], sh[name + ".b"], sh[name + ".alpha"] = (D,), (D,), ()

    norm("final.norm")
    for l, layer in enumerate(cfg["layers"]):
        p, m = f"l{l}.", layer["mixer"]
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        norm(p + "norm1")
        if layer["type"] == "latent_attention_2":
            sh[p + "mix.dq"], sh[p + "mix.dq.norm"], sh[p + "mix.uq"] = (m["q_rank"], D), (m["q_rank"],), (H * (dn + dr), m["q_rank"])
        else:
            sh[p + "mix.q"], sh[p + "mix.sink"] = (H * (dn + dr), D), (H,)
        sh[p + "mix.dkv"], sh[p + "mix.dkv.norm"] = (R + dr, D), (R,)
        sh[p + "mix.uk"], sh[p + "mix.uv"], sh[p + "mix.o"] = (H * dn, R), (H * dv, R), (D, H * dv)
        subs = [1]
        mlp = layer.get("mlp")
        if mlp is not None:
            subs.append(2)
            norm(p + "norm2")
            if mlp["kind"] == "dense":
                sh[p + "mlp.gate"] = sh[p + "mlp.up"] = (mlp["ff"], D)
                sh[p + "mlp.down"] = (D, mlp["ff"])
            else:
                r = mlp["router"]
                n_out = r["experts"] + int(r.get("identity", 0) or 0)
                for e in range(r["experts"]):
                    sh[p + f"mlp.e{e}.gate"] = sh[p + f"mlp.e{e}.up"] = (mlp["expert"]["ff"], D)
                    sh[p + f"mlp.e{e}.down"] = (D, mlp["expert"]["ff"])
                sh[p + "mlp.router"], sh[p + "mlp.correction"] = (n_out, D), (n_out,)
                if mlp.get("shared"):
                    sh[p + "mlp.shared.gate"] = sh[p + "mlp.shared.up"] = (mlp["shared"]["ff"], D)
                    sh[p + "mlp.shared.down"] = (D, mlp["shared"]["ff"])
        for q in subs if S else []:
            sh[p + f"hc{q}.in"], sh[p + f"hc{q}.out"], sh[p + f"hc{q}.mix"] = (S,), (S,), (S, S)
    return sh


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with the design's tensor names, scaled so that every mechanism matters: gate and up
    projections large enough to reach the clamp, router rows that spread the choice, corrections that overturn
    some of it, sinks of order one, stream weights away from 0 / 1."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(cfg).items():
        x = torch.randn(tuple(shape), generator=g)
        leaf = name.split(".", 1)[1] if name[0] == "l" and name[1].isdigit() else name
        if leaf.endswith(".alpha"):
            x = 0.6 + 0.1 * x
        elif leaf.endswith("norm.b") or leaf in ("norm1.b", "norm2.b"):
            x = 0.2 * x
        elif leaf.endswith("norm") or leaf in ("norm1", "norm2"):
            x = 1.0 + 0.2 * x
        elif leaf.startswith("hc") and leaf.endswith(".mix"):
            x = 0.7 * torch.eye(shape[0]) + 0.2 * x
        elif leaf.startswith("hc"):
            x = 0.8 + 0.3 * x
        elif leaf == "mix.sink":
            x = 1.5 * x
        elif leaf == "mlp.correction":
            x = 0.1 * x
        elif leaf == "mlp.router":
            x = 3.0 * x / math.sqrt(shape[-1])
        elif leaf.endswith(".gate") or leaf.endswith(".up"):
            x = 2.0 * x / math.sqrt(shape[-1])
        elif leaf != "embed":
            x = x / math.sqrt(shape[-1])
        out[name] = x.to(torch.bfloat16)
    return out
