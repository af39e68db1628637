"""Small random Mabidra checkpoints for the tests: a config dict, a tensor dict in the checkpoint's naming, and a writer."""
import json
import os

import torch


def attn(heads=4, kv_heads=2, dim=6, vdim=10, scale=None, bias_max=11, rows=8, coef=0.4, every=3):
    """`rows` (the bias table's length) is not a config entry: it is the table's shape"""
    return {"type": "attention", "rows": rows,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5, "bias_max": bias_max,
                      "q_temp": {"coef": coef, "every": every}}}


def gla(heads=3, dim=10, vdim=7, tau=4.0, rank=5):
    return {"type": "gla", "rank": rank, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=12, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, vocab=50, width=24, groups=3, eps=1e-5, emb_scale=0.7, loop=None):
    """layers: [(mixer description from attn() / gla(), feed-forward or None)]; returns (config.json dict, shapes the weights need)"""
    cfg = {"architecture": "Mabidra", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "embedding": {"scale": emb_scale},
           "layers": [{"type": m["type"], "mixer": m["mixer"], "mlp": f} for m, f in layers]}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    extra = [{"rows": m.get("rows"), "rank": m.get("rank")} for m, _ in layers]
    return cfg, extra


def weights(cfg_extra, seed=0, dtype=torch.bfloat16):
    cfg, extra = cfg_extra
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    rn = lambda *s, k=1.0: torch.randn(*s, generator=g) * k
    lin = lambda o, i, s=1.0: rn(o, i, k=s / i ** 0.5)
    nw = lambda n: 1 + 0.2 * rn(n)
    w = {"embed": rn(cfg["vocab"], D), "final.norm": nw(D), "head": lin(cfg["vocab"], D)}
    if "loop" in cfg:
        w["loop.in"], w["loop.step"] = lin(D, 2 * D, 1.4), rn(cfg["loop"]["times"], D, k=0.5)
    for i, (l, x) in enumerate(zip(cfg["layers"], extra)):
        m, p = l["mixer"], f"l{i}."
        w[p + "norm1"], w[p + "norm1b"] = nw(D), nw(D)
        if l["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"], w[p + "mix.o"] = lin(H * d, D), lin(G * d, D), lin(G * dv, D), lin(H, D, 2.0), lin(D, H * dv, 0.5)
            w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"], w[p + "mix.o.b"] = rn(H * d, k=0.3), rn(G * d, k=0.3), rn(G * dv, k=0.3), rn(D, k=0.3)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = nw(d) * 1.5, nw(d) * 1.5
            w[p + "mix.rel"], w[p + "mix.pb"] = rn(x["rows"], H, k=1.5), rn(H) - 1.0
        else:
            H, d, dv, r = m["heads"], m["dim"], m["vdim"], x["rank"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"], w[p + "mix.o"] = lin(H * d, D, 2.0), lin(H * d, D), lin(H * dv, D), lin(H * dv, D, 2.0), lin(D, H * dv)
            w[p + "mix.a1"], w[p + "mix.a2"], w[p + "mix.a2.b"], w[p + "mix.norm"] = lin(r, D), lin(H * d, r, 2.0), rn(H * d) + 1.0, nw(dv)
        f = l["mlp"]
        if f is None:
            continue
        w[p + "norm2"], w[p + "norm2b"] = nw(D), nw(D)
        if f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"] = lin(f["ff"], D, 1.5), lin(D, f["ff"]), rn(2)
        else:
            w[p + "mlp.router"], w[p + "mlp.router.b"] = lin(f["router"]["experts"], D, 3.0), rn(f["router"]["experts"], k=0.5)
            for e in range(f["router"]["experts"]):
                w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(f["expert"]["ff"], D, 2.0), lin(D, f["expert"]["ff"], 2.0)
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def save(path, cfg_extra, w):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg_extra[0], f)
    save_file(w, os.path.join(path, "model.safetensors"))
    return str(path)
