"""Small random Lekapel checkpoints for the tests: a config dict, a tensor dict in the checkpoint's naming, and a writer."""
import json
import os

import torch


def mixer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=20, q_rank=12, window=5, base=100.0, rot_dims=None, scale=None):
    d = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        d["mask"] = {"size": window}
    return d


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=12, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, vocab=50, width=24, groups=3, eps=1e-5, residual_mult=0.6, logit_scale=0.8):
    return {"architecture": "Lekapel", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "residual_mult": residual_mult,
            "logit_scale": logit_scale, "layers": [{"type": "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


def weights(cfg, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    lin = lambda o, i, s=1.0: (torch.randn(o, i, generator=g) * s / i ** 0.5)
    w = {"embed": torch.randn(cfg["vocab"], D, generator=g), "final.norm": 1 + 0.2 * torch.randn(D, generator=g), "head": lin(cfg["vocab"], D)}
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        w[p + "norm1"] = 1 + 0.2 * torch.randn(D, generator=g)
        w[p + "shift"] = torch.rand(D, generator=g)
        w[p + "mix.dq"], w[p + "mix.dq.norm"], w[p + "mix.uq"] = lin(Q, D), 1 + 0.2 * torch.randn(Q, generator=g), lin(H * (dn + dr), Q, 2.0)
        w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = lin(R + dr, D, 2.0), 1 + 0.2 * torch.randn(R, generator=g)
        w[p + "mix.uk"], w[p + "mix.uv"] = lin(H * dn, R, 2.0), lin(H * dv, R)
        w[p + "mix.sink"] = torch.randn(H, generator=g)
        w[p + "mix.g"], w[p + "mix.o"] = lin(H * dv, D), lin(D, H * dv)
        f = l["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"], w[p + "mlp.act"] = lin(f["ff"], D), lin(D, f["ff"]), torch.randn(4, generator=g)
        else:
            w[p + "mlp.router"] = lin(f["router"]["experts"], D, 3.0)
            for e in range(f["router"]["experts"]):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(f["expert"]["ff"], D, 2.0), lin(f["expert"]["ff"], D, 2.0), lin(D, f["expert"]["ff"], 2.0)
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def save(path, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(w, os.path.join(path, "model.safetensors"))
    return str(path)
