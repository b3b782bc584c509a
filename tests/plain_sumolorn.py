"""A plain, slow implementation of the Sumolorn decoder: whole sequences, float64, no cache, no
state carried between calls, one function per mechanism.  It shares no code with the package; the
tests compare the engine with it.

Notation: x [T, w] is the residual stream of one sequence, p = 0..T-1 the positions.  A layer is
x <- x + mix(N1(x)), then (unless it has no feed-forward) x <- x + ff(N2(x)), with
N(u) = u / sqrt(mean(u^2) + eps) * (1 + g).  The layers ``loop.start .. loop.stop - 1`` run
``loop.times`` times in a row with the same weights.
"""

from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------ norms
def rms_norm(x, w, eps, one_plus: bool = False):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * (1.0 + w) if one_plus else y * w


# --------------------------------------------------------------- rotation
def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """f_i = base^(-2i/dims); with ``scaling`` the long wavelengths are stretched: a frequency whose
    wavelength exceeds original/low is divided by factor, one below original/high is kept, and in
    between the two are blended linearly in original/wavelength."""
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(f.numel()):
        wl = 2.0 * math.pi / float(f[i])
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[i] = f[i] / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate_halves(x, pos, dims: int, freq):
    """x [T, heads, D]: among the first ``dims`` elements of a head, element i turns with element
    i + dims/2 by pos * freq[i]."""
    half = dims // 2
    a = pos.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def rotate_pairs(x, pos, dims: int, freq):
    """x [T, heads, D]: among the first ``dims`` elements, element 2i turns with element 2i + 1."""
    a = pos.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# -------------------------------------------------------------- attention
def visible(T: int, window: Optional[int]):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & (i - j < window)
    return m


def softmax_attention(q, k, v, scale: float, window: Optional[int] = None, softcap: Optional[float] = None,
                      sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].  Query head h reads kv head h // (H/G).
    score = q.k scale, then cap tanh(score / cap); the softmax's denominator also holds
    exp(sink_h), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap is not None:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~visible(T, window)[None], -math.inf)
    if sink is not None:
        s = torch.cat([s, sink.to(F64)[:, None, None].expand(H, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    if sink is not None:
        p = p[..., :T]
    return torch.einsum("hij,jhd->ihd", p, vv)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_{t - taps + 1 + j}, zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros((taps - 1, C), dtype=F64), u])
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j][None, :]
    return y


# ------------------------------------------------------- gated recurrence
def gated_linear_attention(q, k, v, alpha):
    """S_t = diag(alpha_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head; q, k, alpha [T, H, D],
    v [T, H, Dv]."""
    T, H, D = q.shape
    S = torch.zeros((H, D, v.shape[-1]), dtype=F64)
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + torch.einsum("hd,he->hde", k[t], v[t])
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    return torch.stack(out)


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------- mixers
def _w(W, name):
    return W[name].to(F64)


def attention_mixer(h, pos, m: dict, W, pre: str, eps: float):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ _w(W, pre + ".q").T)
    k = (h @ _w(W, pre + ".k").T)
    v = (h @ _w(W, pre + ".v").T)
    if m.get("conv"):
        q, k, v = (short_conv(t, _w(W, f"{pre}.{n}.conv")) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        f = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_halves(q, pos, rot["dims"], f), rotate_halves(k, pos, rot["dims"], f)
    if m.get("unit_qk"):
        q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    sink = W.get(pre + ".sink")
    o = softmax_attention(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), m.get("softcap"), sink)
    if pre + ".g" in W:
        o = o * torch.sigmoid(h @ _w(W, pre + ".g").T)[:, :, None]
    return o.reshape(T, H * Dv) @ _w(W, pre + ".o").T


def latent_mixer(h, pos, m: dict, W, pre: str, eps: float):
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if pre + ".dq" in W:
        cq = rms_norm(h @ _w(W, pre + ".dq").T, _w(W, pre + ".dq.norm"), eps)
        q = cq @ _w(W, pre + ".uq").T
    else:
        q = h @ _w(W, pre + ".q").T
    q = q.view(T, H, D + Dr)
    dkv = h @ _w(W, pre + ".dkv").T
    c = rms_norm(dkv[:, :R], _w(W, pre + ".dkv.norm"), eps)
    f = scaled_frequencies(Dr, m["rot"]["base"], m["rot"].get("scaling"))
    kr = rotate_pairs(dkv[:, None, R:], pos, Dr, f)                      # [T, 1, Dr]
    qr = rotate_pairs(q[..., D:], pos, Dr, f)
    ku = (c @ _w(W, pre + ".uk").T).view(T, H, D)
    vv = (c @ _w(W, pre + ".uv").T).view(T, H, Dv)
    qq = torch.cat([q[..., :D], qr], dim=-1)
    kk = torch.cat([ku, kr.expand(T, H, Dr)], dim=-1)
    o = softmax_attention(qq, kk, vv, m["scale"], (m.get("mask") or {}).get("size"), None, W.get(pre + ".sink"))
    if pre + ".g" in W:
        o = o * torch.sigmoid(h @ _w(W, pre + ".g").T)[:, :, None]
    return o.reshape(T, H * Dv) @ _w(W, pre + ".o").T


def gated_decay_mixer(h, m: dict, W, pre: str, eps: float):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ _w(W, pre + ".q").T).view(T, H, D) * D ** -0.5
    k = (h @ _w(W, pre + ".k").T).view(T, H, D)
    v = (h @ _w(W, pre + ".v").T).view(T, H, Dv)
    z = (h @ _w(W, pre + ".a1").T) @ _w(W, pre + ".a2").T + _w(W, pre + ".a2.b")
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, D)
    o = gated_linear_attention(q, k, v, alpha)
    o = rms_norm(o, _w(W, pre + ".norm"), eps).reshape(T, H * Dv)
    return (o * silu(h @ _w(W, pre + ".g").T)) @ _w(W, pre + ".o").T


def parallel_mixer(h, pos, m: dict, W, pre: str, eps: float):
    left = attention_mixer(h, pos, dict(m["left"], unit_qk=True), W, pre + ".left", eps)
    right = gated_decay_mixer(h, m["right"], W, pre + ".right", eps)
    return 0.5 * (rms_norm(left, _w(W, pre + ".left.out"), eps) + rms_norm(right, _w(W, pre + ".right.out"), eps))


# ----------------------------------------------------------- feed-forward
def clamped_feed_forward(h, mlp: dict, W, pre: str):
    lim = mlp["limit"]
    g = (h @ _w(W, pre + ".gate").T).clamp(max=lim)
    u = (h @ _w(W, pre + ".up").T).clamp(min=-lim, max=lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _w(W, pre + ".down").T


# ------------------------------------------------------------------ model
def layer_runs(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, W: Dict[str, torch.Tensor], ids: List[int], streams: Optional[list] = None):
    """Logits [T, vocab] float64 of one sequence; ``streams`` (a list) receives the stream after
    every layer run."""
    eps = cfg["norm"]["eps"]
    x = _w(W, "embed")[torch.tensor(ids)]
    pos = torch.arange(len(ids))
    for i in layer_runs(cfg):
        L = cfg["layers"][i]
        pre = f"l{i}"
        h = rms_norm(x, _w(W, pre + ".norm1"), eps, one_plus=True)
        if L["type"] == "attention":
            y = attention_mixer(h, pos, L["mixer"], W, pre + ".mix", eps)
        elif L["type"] == "latent_attention":
            y = latent_mixer(h, pos, L["mixer"], W, pre + ".mix", eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(h, pos, L["mixer"], W, pre + ".mix", eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp"):
            x = x + clamped_feed_forward(rms_norm(x, _w(W, pre + ".norm2"), eps, one_plus=True), L["mlp"], W,
                                         pre + ".mlp")
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, _w(W, "final.norm"), eps, one_plus=True)
    return (x @ _w(W, "head").T) * cfg.get("logit_scale", 1.0)


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
