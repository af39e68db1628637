"""TEST-ONLY plain restatement of the Mabidra decoder, one function per mechanism, float64 (or float32) torch on the CPU.

Nothing here is imported by the product path and nothing of the product path is imported here.  Every function works on one
sequence `[tokens, features]`; `Model.forward` runs a token range over explicit Python state (lists of cached keys and values,
one state matrix per head), with no paging and no batching, token by token where a recurrence is involved.

Notation: `T` tokens, `D` model width, `H` query heads, `G` key/value heads, `d` query/key size and `dv` value size per head.
"""
from __future__ import annotations

import math

import torch

from .lekapel_oracle import read_safetensors  # noqa: F401  (the same file format)


def grouped_rms_norm(x, w, groups, eps):
    """every one of `groups` equal consecutive parts of a row is divided by sqrt(mean(part^2) + eps); the row then times w"""
    out = []
    for part in x.chunk(groups, dim=-1):
        out.append(part / torch.sqrt((part * part).mean(-1, keepdim=True) + eps))
    return torch.cat(out, -1) * w


def head_rms_norm(x, w, eps):
    """x [..., n] over its last axis, one weight vector for all heads"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def distance_bucket(n, rows, reach):
    """bucket of the distance n >= 0 in a table of `rows` rows: itself below rows // 2, then logarithmic steps that arrive at
    the last row when n = reach, and the last row from there on"""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def query_temperature(pos, coef, every):
    """1 + coef * ln(floor((pos + 1) / every) + 1) for integer positions"""
    return 1.0 + coef * torch.log(torch.div(pos + 1, every, rounding_mode="floor").double() + 1.0)


def sigmoid_attention(q, k, v, qpos, kpos, scale, rel, pb, reach):
    """q [T, H, d], k [N, G, d], v [N, G, dv]; every visible key (kpos <= qpos) weighs sigmoid(scale q.k + rel[bucket][h] + pb[h]);
    the weights are not normalised.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        for h in range(H):
            g = h // (H // G)
            for j in range(k.shape[0]):
                n = int(qpos[i]) - int(kpos[j])
                if n < 0:
                    continue
                s = (q[i, h] * k[j, g]).sum() * scale + rel[distance_bucket(n, rel.shape[0], reach), h] + pb[h]
                out[i, h] += torch.sigmoid(s) * v[j, g]
    return out


def sigmoid_attention_fast(q, k, v, qpos, kpos, scale, rel, pb, reach):
    """the same sums as `sigmoid_attention`, written with matrix products (for long test sequences)"""
    T, H, _ = q.shape
    G = k.shape[1]
    n = qpos[:, None] - kpos[None, :]
    bucket = torch.tensor([distance_bucket(x, rel.shape[0], reach) for x in range(int(n.max()) + 1)])
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale + rel[bucket[n.clamp(min=0)], h] + pb[h]
        out[:, h] = (torch.sigmoid(s) * (n >= 0)) @ v[:, g]
    return out


def attention_mixer(h, pos, past, W, m, eps, fast=True):
    """h [T, D] -> ([T, D], new past).  past = (keys [N, G, d], values [N, G, dv], positions [N]) of the earlier tokens."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = head_rms_norm((h @ W["q"].T + W["q.b"]).reshape(T, H, d), W["q.norm"], eps)
    k = head_rms_norm((h @ W["k"].T + W["k.b"]).reshape(T, G, d), W["k.norm"], eps)
    v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"]).to(h.dtype)[:, None, None]
    keys, values, kpos = torch.cat([past[0], k]), torch.cat([past[1], v]), torch.cat([past[2], pos])
    attend = sigmoid_attention_fast if fast else sigmoid_attention
    o = attend(q, keys, values, pos, kpos, m["scale"], W["rel"], W["pb"], m["bias_max"])
    o = o * torch.sigmoid(h @ W["g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W["o"].T + W["o.b"], (keys, values, kpos)


def gla_recurrence(q, k, v, a, S):
    """q, k, a [T, H, d], v [T, H, dv], S [H, d, dv]: S <- a_t (rows) * S + k_t v_t^T, o_t = S^T q_t.  Returns (o [T, H, dv], S)."""
    o = []
    for t in range(q.shape[0]):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o.append((S * q[t][:, :, None]).sum(1))
    return torch.stack(o), S


def gla_mixer(h, S, W, m, eps):
    """h [T, D], S [H, d, dv] -> ([T, D], new S)"""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, d) / math.sqrt(d)
    k = (h @ W["k"].T).reshape(T, H, d)
    v = (h @ W["v"].T).reshape(T, H, dv)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    a = torch.sigmoid(z).pow(1.0 / m["tau"]).reshape(T, H, d)
    o, S = gla_recurrence(q, k, v, a, S)
    o = head_rms_norm(o, W["norm"], eps).reshape(T, H * dv)
    g = h @ W["g"].T
    return (o * g * torch.sigmoid(g)) @ W["o"].T, S


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    neg = z.clamp(max=0.0)
    return torch.where(z > 0, sp(p) * z * z + z / 2, (0.5 + sp(q)) * (torch.exp(neg) - 1 - neg) + neg / 2)


def xielu_mlp(h, up, down, pq):
    return xielu(h @ up.T, pq[0], pq[1]) @ down.T


def topk_softmax_router(h, router, bias, top):
    """(ids [T, top], weights [T, top]): the `top` largest of W h + b, soft-max over those only"""
    val, idx = (h @ router.T + bias).topk(top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def relu2_moe_mlp(h, W, top):
    idx, w = topk_softmax_router(h, W["router"], W["router.b"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += w[t, j] * (torch.relu(W[f"e{e}.up"] @ h[t]).square() @ W[f"e{e}.down"].T)
    return out


class Model:
    def __init__(self, config, tensors, dtype=torch.float64):
        self.c, self.dtype = config, dtype
        self.W = {k: v.to(dtype) for k, v in tensors.items()}
        n, lp = len(config["layers"]), config.get("loop")
        if lp is None:
            self.runs = [(i, None) for i in range(n)]
        else:
            self.runs = [(i, None) for i in range(lp["start"])]
            for t in range(lp["times"]):
                self.runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
            self.runs += [(i, None) for i in range(lp["stop"], n)]

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.W.items() if k.startswith(prefix)}

    def new_state(self):
        st = {"pos": 0, "runs": []}
        for i, _ in self.runs:
            l = self.c["layers"][i]
            m = l["mixer"]
            if l["type"] == "attention":
                st["runs"].append((torch.zeros(0, m["kv_heads"], m["dim"], dtype=self.dtype), torch.zeros(0, m["kv_heads"], m["vdim"], dtype=self.dtype),
                                   torch.zeros(0, dtype=torch.long)))
            else:
                st["runs"].append(torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=self.dtype))
        return st

    def forward(self, tokens, state, trace=None):
        """logits [len(tokens), vocab] of the next tokens of ONE sequence; `state` is advanced"""
        c, W = self.c, self.W
        eps, groups = c["norm"]["eps"], c["norm"]["groups"]
        norm = lambda x, key: grouped_rms_norm(x, W[key], groups, eps)
        pos = torch.arange(state["pos"], state["pos"] + len(tokens))
        x0 = W["embed"][torch.tensor(tokens)] * c["embedding"]["scale"]
        x = x0
        for r, (i, opens) in enumerate(self.runs):
            if opens is not None:
                x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][opens]
            l, p = c["layers"][i], f"l{i}."
            if l["type"] == "attention":
                y, state["runs"][r] = attention_mixer(norm(x, p + "norm1"), pos, state["runs"][r], self.sub(p + "mix."), l["mixer"], eps)
            else:
                y, state["runs"][r] = gla_mixer(norm(x, p + "norm1"), state["runs"][r], self.sub(p + "mix."), l["mixer"], eps)
            x = x + norm(y, p + "norm1b")
            f = l["mlp"]
            if f is not None:
                h = norm(x, p + "norm2")
                y = xielu_mlp(h, W[p + "mlp.up"], W[p + "mlp.down"], W[p + "mlp.act"]) if f["kind"] == "dense" else relu2_moe_mlp(h, self.sub(p + "mlp."), f["router"]["top"])
                x = x + norm(y, p + "norm2b")
            if trace is not None:
                trace.append(x.clone())
        state["pos"] += len(tokens)
        return norm(x, "final.norm") @ W["head"].T
