"""A plain, slow implementation of the Zimupel decoder: whole sequences, float64, no cache, no
state carried between calls, one function per mechanism.  It shares no code with the package; the
tests compare the engine with it.

Notation: X [n, T, w] are the n residual streams of one sequence (n = 1 without hyper-connections),
p = 0..T-1 the positions.  A sublayer f with norm N reads u = sum_s a_s X_s and writes
X_t <- sum_s M[s, t] X_s + b_t f(N(u)); without hyper-connections that is x <- x + f(N(x)).
"""

from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------ norms
def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


# --------------------------------------------------------------- rotation
def rotate_halves(x, pos, dims: int, base: float):
    """x [T, heads, D]: among the first ``dims`` elements of every head, element i is rotated with
    element i + dims/2 by the angle pos * base^(-2i/dims); the rest pass."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    a = pos.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------- recurrences with a decay
def decayed_sum(q, k, v, decay):
    """o_t = sum_{j <= t} decay_h^(t-j) (q_t . k_j) v_j per head: the closed form of
    S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D], v [T, H, Dv]."""
    T = q.shape[0]
    i = torch.arange(T, dtype=F64)[:, None]
    j = torch.arange(T, dtype=F64)[None, :]
    d = torch.tensor(list(decay), dtype=F64)
    w = torch.where(j <= i, d[:, None, None] ** (i - j).clamp(min=0), torch.zeros((), dtype=F64))   # [H, T, T]
    s = torch.einsum("ihd,jhd->hij", q, k) * w
    return torch.einsum("hij,jhd->ihd", s, v)


def decayed_sum_stepwise(q, k, v, decay):
    """The same by the recurrence itself, a token at a time (a check of ``decayed_sum``)."""
    T, H, D = q.shape
    S = torch.zeros((H, D, v.shape[-1]), dtype=F64)
    d = torch.tensor(list(decay), dtype=F64)[:, None, None]
    out = []
    for t in range(T):
        S = d * S + torch.einsum("hd,he->hde", k[t], v[t])
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    return torch.stack(out)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------- mixers
def retention_mixer(h, W, pre: str, m: dict, eps: float, pos):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).view(T, H, D)
    k = (h @ W[pre + "k"].T).view(T, H, D)
    v = (h @ W[pre + "v"].T).view(T, H, Dv)
    rot = m.get("rot")
    if rot:
        q = rotate_halves(q, pos, rot["dims"], rot["base"])
        k = rotate_halves(k, pos, rot["dims"], rot["base"])
    k = k * D ** -0.5
    o = rms_norm(decayed_sum(q, k, v, m["decay"]), None, eps)          # per head, no weight
    return (o.reshape(T, H * Dv) * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def lightning_mixer(h, W, pre: str, m: dict, eps: float):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[pre + "q"].T).view(T, H, D)
    k = silu(h @ W[pre + "k"].T).view(T, H, D)
    v = silu(h @ W[pre + "v"].T).view(T, H, Dv)
    o = decayed_sum(q, k, v, m["decay"]).reshape(T, H * Dv)
    o = rms_norm(o, W[pre + "norm"], eps)                              # over all heads together
    return (o * torch.sigmoid(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def causal_softmax(q, k, v, scale):
    """q, k [T, H, D], v [T, H, Dv], one key head per query head."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v)


def differential_lambda(W, pre: str, diff: float):
    return (math.exp(float((W[pre + "lq1"] * W[pre + "lk1"]).sum()))
            - math.exp(float((W[pre + "lq2"] * W[pre + "lk2"]).sum())) + diff)


def differential_keys_values(h, W, pre: str, m: dict):
    """(k [T, G, 2, D], v [T, G, Dv]) of a layer that has projections of its own."""
    T = h.shape[0]
    G = m.get("kv_heads", m["heads"])
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).view(T, G, 2, m["dim"])
    v = (h @ W[pre + "v"].T + W[pre + "v.b"]).view(T, G, m["vdim"])
    return k, v


def differential_mixer(h, W, pre: str, m: dict, eps: float, kv):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads", H)
    k, v = kv
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).view(T, H, 2, D)
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)                               # query head h uses kv head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    a1 = causal_softmax(q[:, :, 0], kk[:, :, 0], vv, m["scale"])
    a2 = causal_softmax(q[:, :, 1], kk[:, :, 1], vv, m["scale"])
    lam = differential_lambda(W, pre, m["diff"])
    o = rms_norm(a1 - lam * a2, None, eps) * (1.0 - m["diff"])
    return o.reshape(T, H * Dv) @ W[pre + "o"].T


# ---------------------------------------------------------- feed-forwards
def dense_ff(h, W, pre: str, act):
    return (act(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def route(z, correction, r: dict):
    """(chosen experts [T, top], weights [T, top]) from router logits z [T, E]."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    c = s + correction
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        cg = c.view(-1, n, per)
        gscore = cg.topk(min(2, per), dim=-1).values.sum(-1)           # a group: its two best
        best = gscore.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        c = torch.where(allowed[:, :, None].expand_as(cg), cg,
                        torch.full_like(cg, float("-inf"))).reshape(-1, E)
    ids = c.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20)


def routed_ff(h, W, pre: str, mlp: dict):
    r = mlp["router"]
    ids, w = route(h @ W[pre + "router"].T, W[pre + "correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            out[t] += w[t, j] * dense_ff(h[t:t + 1], W, f"{pre}e{e}.", silu)[0]
    return out


# ------------------------------------------------------------------ model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] float64 of one sequence (and the summed streams after every layer)."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = rms_norm(W["embed"][torch.tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    n = cfg.get("streams")
    X = x[None].repeat(n or 1, 1, 1)
    kv_of: Dict[int, tuple] = {}
    after = []

    def sublayer(X, i, q, f):
        norm_w = W[f"l{i}.norm{q}"]
        if n is None:
            return X + f(rms_norm(X[0], norm_w, eps))[None]
        a, b, M = W[f"l{i}.hc{q}.in"], W[f"l{i}.hc{q}.out"], W[f"l{i}.hc{q}.mix"]
        y = f(rms_norm(torch.einsum("s,stw->tw", a, X), norm_w, eps))
        return torch.einsum("sr,stw->rtw", M, X) + b[:, None, None] * y[None]

    for i, layer in enumerate(cfg["layers"]):
        kind, m, pre = layer["type"], layer["mixer"], f"l{i}.mix."
        if kind == "retention":
            f = lambda h: retention_mixer(h, W, pre, m, eps, pos)
        elif kind == "lightning":
            f = lambda h: lightning_mixer(h, W, pre, m, eps)
        else:
            def f(h):
                if "kv_from" in m:
                    kv = kv_of[m["kv_from"]]
                else:
                    kv = kv_of[i] = differential_keys_values(h, W, pre, m)
                return differential_mixer(h, W, pre, m, eps, kv)
        X = sublayer(X, i, 1, f)
        mlp = layer.get("mlp")
        if mlp:
            mp = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                X = sublayer(X, i, 2, lambda h: dense_ff(h, W, mp, gelu_tanh))
            else:
                X = sublayer(X, i, 2, lambda h: routed_ff(h, W, mp, mlp))
        after.append(X.sum(0))
    x = rms_norm(X.sum(0), W["final.norm"], eps)
    z = x @ W["head"].T
    if cfg.get("logit_scale") is not None:
        z = z * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * torch.tanh(z / cap)
    return (z, torch.stack(after)) if return_layers else z


# ----------------------------------------------------------- model folders
_DT = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
       "I32": (torch.int32, 4), "I64": (torch.int64, 8)}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[e["dtype"]]
        lo, hi = e["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=dt).reshape(e["shape"]).clone()
    return out


def load_folder(folder: str):
    with open(f"{folder}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{folder}/model.safetensors")


def greedy(cfg: dict, W: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """``n_new`` tokens by arg-max, the whole sequence recomputed for every token."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward(cfg, W, ids)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out
