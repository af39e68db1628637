"""TEST-ONLY plain restatement of the Lekapel decoder, one function per mechanism, float32 (or float64) torch on the CPU.

Nothing here is imported by the product path and nothing of the product path is imported here.  Every function works on
one sequence `[tokens, features]`; `forward` runs a whole model token range by token range over explicit Python state
(lists of cached latents, previous normed rows), with no paging and no batching.

Notation: `T` tokens, `D` model width, `H` heads, `dn` un-rotated and `dr` rotated query/key sizes per head, `dv` value size,
`R` latent size.
"""
from __future__ import annotations

import json
import math
import struct

import torch


def read_safetensors(path):
    """{name: tensor} from one safetensors file: u64 header length, JSON header, raw little-endian data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        blob = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(blob[lo:hi]), dtype=kinds[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def grouped_rms_norm(x, w, groups, eps):
    """x [T, D] is cut into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps); then * w."""
    T, D = x.shape
    p = x.reshape(T, groups, D // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, D) * w


def token_shift(h, prev, mu):
    """Row t becomes h_t + (h_{t-1} - h_t) * mu, with the un-shifted rows on the right-hand side; `prev` stands before row 0
    (zeros at the start of a sequence).  Returns (shifted, last un-shifted row)."""
    before = torch.cat([prev[None], h[:-1]], 0)
    return h + (before - h) * mu, h[-1]


def rotate_interleaved(x, pos, base, dims):
    """x [T, ..., d]: the pairs (2i, 2i+1), i < dims/2, are turned by the angle pos * base^(-2i/dims); the rest passes."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = (pos.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)).to(x.dtype)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, qpos, kpos, scale, sink, window):
    """q [Tq, H, dq], k [Tk, H, dq], v [Tk, H, dv]; query at position i sees key at position j when 0 <= i - j < window
    (`window` None: every j <= i).  The soft-max denominator holds one extra term exp(sink_h) that has no value."""
    s = torch.einsum("qhd,khd->hqk", q, k) * scale
    d = qpos[:, None] - kpos[None, :]
    ok = d >= 0
    if window is not None:
        ok = ok & (d < window)
    s = s.masked_fill(~ok[None], float("-inf"))
    m = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - m[..., None])
    den = e.sum(-1) + torch.exp(sink[:, None] - m)
    return torch.einsum("hqk,khd->qhd", e / den[..., None], v)


def latent_attention(h, pos, past, W, m, eps):
    """One mixer call over new rows h [T, D] at positions pos [T]; `past` = (latents [L, R], rotated key parts [L, dr],
    positions [L]) of the earlier tokens.  Returns (output [T, D], new past)."""
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    cq = h @ W["dq"].T
    cq = cq / torch.sqrt((cq * cq).mean(-1, keepdim=True) + eps) * W["dq.norm"]
    q = (cq @ W["uq"].T).reshape(-1, H, dn + dr)
    kv = h @ W["dkv"].T
    c, kr = kv[:, :R], kv[:, R:]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * W["dkv.norm"]
    q = torch.cat([q[..., :dn], rotate_interleaved(q[..., dn:], pos, rot["base"], rot["dims"])], -1)
    kr = rotate_interleaved(kr, pos, rot["base"], rot["dims"])
    c_all, kr_all, p_all = torch.cat([past[0], c]), torch.cat([past[1], kr]), torch.cat([past[2], pos])
    kn = (c_all @ W["uk"].T).reshape(-1, H, dn)
    v = (c_all @ W["uv"].T).reshape(-1, H, dv)
    k = torch.cat([kn, kr_all[:, None, :].expand(-1, H, -1)], -1)
    window = (m.get("mask") or {}).get("size")
    o = sink_softmax_attention(q, k, v, pos, p_all, m["scale"], W["sink"], window).reshape(-1, H * dv)
    o = o * torch.sigmoid(h @ W["g"].T)
    return o @ W["o"].T, (c_all, kr_all, p_all)


def poly_norm_mlp(h, up, down, coef, eps):
    """down . (a N(z) + b N(z^2) + c N(z^3) + e), z = up . h, N(y) = y / sqrt(mean(y^2) + eps) over the ff values of a token."""
    z = h @ up.T
    n = lambda y: y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (coef[0] * n(z) + coef[1] * n(z * z) + coef[2] * n(z * z * z) + coef[3]) @ down.T


def softmax_topk_router(h, router, top):
    """scores = softmax(router . h) over all experts; the `top` largest are kept with their scores as weights (no re-scaling)."""
    s = torch.softmax(h @ router.T, -1)
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def moe_mlp(h, W, experts, top):
    idx, w = softmax_topk_router(h, W["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = h[t] @ W[f"e{e}.gate"].T
            out[t] += w[t, j] * ((a * torch.sigmoid(a) * (h[t] @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T)
    return out


class Model:
    def __init__(self, config, tensors, dtype=torch.float32):
        self.cfg = config
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.dtype = dtype

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        D = self.cfg["width"]
        st = []
        for layer in self.cfg["layers"]:
            m = layer["mixer"]
            st.append({"prev": torch.zeros(D, dtype=self.dtype),
                       "past": (torch.zeros(0, m["kv_rank"], dtype=self.dtype), torch.zeros(0, m["rot_dim"], dtype=self.dtype),
                                torch.zeros(0, dtype=torch.long))})
        return {"layers": st, "n": 0}

    def forward(self, tokens, state, trace=None):
        """Runs `tokens` (a list) after whatever `state` holds; returns logits [T, vocab]."""
        cfg, eps, groups = self.cfg, self.cfg["norm"]["eps"], self.cfg["norm"]["groups"]
        pos = torch.arange(state["n"], state["n"] + len(tokens))
        x = self.w["embed"][torch.tensor(tokens)]
        for i, layer in enumerate(cfg["layers"]):
            st = state["layers"][i]
            h = grouped_rms_norm(x, self.w[f"l{i}.norm1"], groups, eps)
            hs, st["prev"] = token_shift(h, st["prev"], self.w[f"l{i}.shift"])
            assert layer["type"] == "latent_attention"
            y, st["past"] = latent_attention(hs, pos, st["past"], self.sub(f"l{i}.mix."), layer["mixer"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                W = self.sub(f"l{i}.mlp.")
                if mlp["kind"] == "dense":
                    y = y + poly_norm_mlp(h, W["up"], W["down"], W["act"], eps)
                else:
                    y = y + moe_mlp(h, W, mlp["router"]["experts"], mlp["router"]["top"])
            x = x + cfg["residual_mult"] * y
            if trace is not None:
                trace.append(x.clone())
        state["n"] += len(tokens)
        x = grouped_rms_norm(x, self.w["final.norm"], groups, eps)
        return (x @ self.w["head"].T) * cfg["logit_scale"]
