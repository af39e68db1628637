"""Lekapel through the framework (registry, loader, paged state cache, scheduler, engine, CUDA operators) against the plain
restatement in oracle/lekapel_oracle.py, on small random checkpoints made here.  CPU tests cover the host logic."""
import json

import pytest
import torch

import lekapel_util as U
from oracle import lekapel_oracle as O

gpu = pytest.mark.gpu
F32_TOL, BF16_TOL = 3e-4, 6e-2


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def rel_rows(a, b, q=0.8):
    """the q-quantile of the per-row errors: for bf16 runs of whole models, where rounding may flip a close routing choice of
    a few tokens (the restatement routes in float64)"""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float(((a - b).abs().amax(-1) / b.abs().max()).quantile(q))


class DictLoader:
    def __init__(self, w):
        self.w = w

    def load_tensor(self, key, device="cpu"):
        return self.w[key].to(device)


MIXED = [(U.mixer(), U.dense()), (U.mixer(heads=2, dim=6, rot_dim=8, vdim=4, kv_rank=33, q_rank=10, window=7, rot_dims=4), U.moe()),
         (U.mixer(heads=9, dim=4, rot_dim=2, vdim=8, kv_rank=16, q_rank=8, window=None), None), (U.mixer(window=1), U.moe(ff=8, experts=3, top=1))]


def serve(tmp_path, cfg, dtype, seed=0, **engine_kw):
    from ktransformers_b200.models import load_model
    from ktransformers_b200.util.engine import Engine
    w = U.weights(cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / f"ckpt{seed}", cfg, w)
    torch.backends.cuda.matmul.allow_tf32 = False
    model = load_model(path, dtype)
    return Engine(model, **engine_kw), O.Model(cfg, w, torch.float64)


def oracle_logits(om, tokens):
    return om.forward(tokens, om.new_state()).float()


def run_steps(eng, steps):
    """steps: list of lists of (id, tokens, last); every position's logits are asked for; returns {id: [n, V]}"""
    out = {}
    for step in steps:
        lg = eng.step([(i, t, list(range(len(t)))) for i, t, _ in step], [i for i, _, last in step if last]).cpu()
        k = 0
        for i, t, _ in step:
            out.setdefault(i, []).append(lg[k:k + len(t)])
            k += len(t)
    return {i: torch.cat(v) for i, v in out.items()}


def cut(seq_id, tokens, sizes):
    """portions of the given sizes (repeating the last) as single-entry steps"""
    steps, at, k = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(k, len(sizes) - 1)], len(tokens) - at)
        steps.append([(seq_id, tokens[at:at + n], at + n == len(tokens))])
        at, k = at + n, k + 1
    return steps


def toks(n, vocab=50, seed=0):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------------------------------------ host logic (CPU)
def test_config_reads_sizes_per_layer():
    from ktransformers_b200.models.configuration_lekapel import LekapelConfig
    c = LekapelConfig.from_dict(U.config(MIXED, vocab=77, width=36, groups=2, residual_mult=1.0))
    assert (c.vocab, c.width, c.norm_groups, c.residual_mult, len(c.layers)) == (77, 36, 2, 1.0, 4)
    assert c.layers[1].mixer.rot.dims == 4 and c.layers[1].mixer.rot_dim == 8 and c.layers[1].mixer.window == 7
    assert c.layers[2].mixer.window is None and c.layers[2].mlp is None and c.max_window() is None
    assert c.layers[3].mlp.top == 1 and c.layers[3].mlp.experts == 3 and c.layers[0].mlp.kind == "dense"
    assert c.cache_row_widths() == [24, 41, 18, 24]
    assert LekapelConfig.from_dict(U.config(MIXED[:2])).max_window() == 7


def test_registry_picks_the_class_by_config():
    from ktransformers_b200.models import architecture_of, model_class
    assert model_class(architecture_of({"architecture": "Lekapel"})).__name__ == "LekapelForCausalLM"
    assert architecture_of({"architectures": ["DeepseekV3ForCausalLM"]}) == "DeepseekV3ForCausalLM"
    with pytest.raises(ValueError):
        model_class("NoSuchModel")


def test_oracle_portions_equal_whole_prompt(tmp_path):
    cfg = U.config(MIXED)
    w = U.weights(cfg, 3, torch.float32)
    U.save(tmp_path / "m", cfg, w)
    back = O.read_safetensors(str(tmp_path / "m" / "model.safetensors"))
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    om = O.Model(cfg, back, torch.float64)
    t = toks(19)
    whole = oracle_logits(om, t)
    st, parts = om.new_state(), []
    for lo, hi in ((0, 1), (1, 3), (3, 10), (10, 11), (11, 19)):
        parts.append(om.forward(t[lo:hi], st).float())
    assert rel(torch.cat(parts), whole) < 1e-6


def test_paged_cache_reuses_pages_and_slots_and_releases_behind_the_window():
    from ktransformers_b200.models.custom_cache import PagedStateCache
    c = PagedStateCache([6, 4], 8, max_tokens=32, max_slots=2, device="cpu", dtype=torch.float32, page_size=4, window=5)
    total = c.num_pages
    b = c.build_batch([("a", [1, 2, 3, 4, 5, 6], [5]), ("b", [7], [0])])
    assert b.pos.tolist() == [0, 1, 2, 3, 4, 5, 0] and b.slot.tolist() == [0] * 6 + [1]
    assert b.prev_idx.tolist() == [-1, 0, 1, 2, 3, 4, -1] and b.rd_row.tolist() == [-1] * 7
    assert b.wr_row.tolist() == [-1] * 5 + [1, 3] and b.want.tolist() == [5, 6]
    c.commit()
    b = c.build_batch([("a", [9], [])])
    assert b.pos.tolist() == [6] and b.rd_row.tolist() == [1] and b.wr_row.tolist() == [0] and b.prev_idx.tolist() == [-1]
    c.commit()
    # a long sequence with window 5 and pages of 4 never holds more than 3 pages
    for _ in range(80):                                       # far past max_tokens: the page table row is a ring
        c.build_batch([("a", [1], [])])
        c.commit()
        assert total - len(c._free_pages) - 1 <= 3            # (sequence b holds one page)
    used_by_a = {int(c._table_host[0, p % c.max_pages_per_seq]) for p in range(c._first_page[0], (c.length("a") + 3) // 4)}
    c.close("a")
    c.close("b")
    assert len(c._free_pages) == total and len(c._free_slots) == 2
    s = c.open("c")
    c.extend(s, 4)
    assert int(c._table_host[s, 0]) in used_by_a | {int(c._table_host[1, 0])}   # a freed page is handed out again
    assert c.state_rows(s, 0)[0] == -1                                           # a reused slot starts without state
    with pytest.raises(MemoryError):
        c.extend(s, 10_000)


def test_scheduler_mixes_decode_tokens_and_prompt_portions():
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.util.scheduler import Request, Scheduler
    c = PagedStateCache([4], 4, max_tokens=256, max_slots=3, device="cpu", dtype=torch.float32, page_size=4)
    s = Scheduler(c, max_step_tokens=8)
    a, b = Request("a", list(range(5)), 4), Request("b", list(range(11)), 4)
    s.add(a), s.add(b)
    e = s.schedule()
    assert [(x.request.id, len(x.tokens), x.want_last) for x in e] == [("a", 5, True), ("b", 3, False)]
    a.fed, b.fed, a.pending = 5, 3, 42
    e = s.schedule()
    assert [(x.request.id, x.tokens if x.request is a else len(x.tokens), x.want_last) for x in e] == [("a", [42], True), ("b", 7, False)]
    b.fed = 10
    e = s.schedule()
    assert [(x.request.id, len(x.tokens), x.want_last) for x in e] == [("a", 1, True), ("b", 1, True)]


def test_sampler():
    from ktransformers_b200.util.engine import Sampler
    z = torch.tensor([[0.0, 3.0, 1.0], [5.0, 0.0, 0.0]])
    assert Sampler()(z).tolist() == [1, 0]
    assert Sampler(temperature=1.0, top_k=1)(z).tolist() == [1, 0]
    assert Sampler(temperature=1.0, top_p=1e-6)(z).tolist() == [1, 0]


# ------------------------------------------------------------------------------------------------ mechanisms alone (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("groups,width", [(1, 20), (3, 36), (4, 256), (5, 35), (16, 64)])      # 16-byte and element-wise paths
def test_group_norm_and_shift_kernel(dtype, tol, groups, width):
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.operators.norm import KGroupRMSNormShift
    g = torch.Generator().manual_seed(1)
    x, a, b = (torch.randn(7, width, generator=g) for _ in range(3))
    w, mu = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype), torch.rand(width, generator=g).to(dtype)
    op = KGroupRMSNormShift(width, groups, 1e-5, True, dtype=dtype)
    op.load(DictLoader({"n": w, "s": mu}), "n", "s")
    cache = PagedStateCache([4], width, 64, 2, "cuda", dtype=dtype, page_size=4)
    a_d, b_d = a.to(dtype).cuda(), b.cuda()                      # one branch in the compute dtype, one in fp32
    xs = x + 0.6 * (a.to(dtype).float() + b)
    h = O.grouped_rms_norm(xs.double(), w.double(), groups, 1e-5)
    hs, _ = O.token_shift(h, torch.zeros(width, dtype=torch.float64), mu.double())
    # rows 0..3 in one launch, 4 alone, 5..6 together: the shifted rows must not depend on the cut
    outs = []
    for lo, hi in ((0, 4), (4, 5), (5, 7)):
        batch = cache.build_batch([("s", [0] * (hi - lo), [])])
        xo, ho, so = op(x[lo:hi].cuda().contiguous(), a_d[lo:hi].contiguous(), b_d[lo:hi].contiguous(), 0.6, batch, cache.state[0])
        cache.commit()
        outs.append((xo, ho, so))
    assert rel(torch.cat([o[0] for o in outs]), xs) < 1e-6
    assert rel(torch.cat([o[1] for o in outs]), h) < tol and rel(torch.cat([o[2] for o in outs]), hs) < tol


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_poly_norm_mlp(dtype, tol):
    from ktransformers_b200.operators.mlp import KPolyNormMLP
    g = torch.Generator().manual_seed(2)
    up, down, coef = torch.randn(52, 24, generator=g).to(dtype), torch.randn(24, 52, generator=g).to(dtype), torch.tensor([0.7, -0.4, 0.25, 0.1])
    op = KPolyNormMLP(24, 52, 1e-5, dtype=dtype)
    op.load(DictLoader({"up": up, "down": down, "act": coef.to(dtype)}), "")
    h = torch.randn(9, 24, generator=g).to(dtype)
    want = O.poly_norm_mlp(h.double(), up.double(), down.double(), coef.to(dtype).double(), 1e-5)
    assert rel(op(h.cuda()), want) < tol


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("experts,top,ff,width", [(5, 2, 12, 24), (3, 1, 7, 20), (16, 4, 64, 128), (4, 2, 6, 18)])
@pytest.mark.parametrize("tokens", [1, 11, 70])              # per-pair kernels / an expert's rows once for several pairs / grouped GEMMs
def test_softmax_topk_moe(dtype, tol, experts, top, ff, width, tokens):
    from ktransformers_b200.operators.experts import KSoftmaxTopKMoE
    g = torch.Generator().manual_seed(3)
    W = {"router": (torch.randn(experts, width, generator=g) * 0.5).to(dtype)}
    for e in range(experts):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = ((torch.randn(s, generator=g) * 0.3).to(dtype) for s in ((ff, width), (ff, width), (width, ff)))
    op = KSoftmaxTopKMoE(width, ff, experts, top, dtype=dtype)
    op.load(DictLoader(W), "")
    h = torch.randn(tokens, width, generator=g).to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    ids, w = op.router(h.cuda())
    oi, ow = O.softmax_topk_router(h.double(), Wd["router"], top)
    assert torch.equal(ids.cpu().sort(-1).values, oi.sort(-1).values)
    assert rel(w.cpu().sort(-1).values, ow.sort(-1).values) < 1e-5       # the chosen scores themselves: not re-scaled to sum 1
    assert rel(op(h.cuda()), O.moe_mlp(h.double(), Wd, experts, top)) < tol


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,width,tokens", [(4, 2, 16, 24, 13), (3, 3, 7, 20, 5), (16, 4, 64, 128, 40), (2, 1, 33, 9, 9), (32, 8, 40, 64, 2)])
def test_experts_by_expert_kernels_equal_the_per_pair_kernels(dtype, experts, top, ff, width, tokens):
    """many pairs on one expert (more than the kernel stages at once), experts without pairs, 16-byte and element-wise rows: the
    same activations bit for bit, and the same weighted sums up to the order of the lane sums"""
    from ktransformers_b200.operators.experts import KExpertsDense
    g = torch.Generator().manual_seed(11)
    op = KExpertsDense(width, ff, experts, dtype=dtype)
    for p in (op.gate, op.up, op.down):
        p.data.copy_((torch.randn(p.shape, generator=g) * 0.3).to(dtype))
    x = torch.randn(tokens, width, generator=g).to(dtype).cuda()
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)])
    ids[: tokens // 2] = ids[0]                      # half of the tokens share their experts
    ids, w = ids.cuda(), torch.rand(tokens, top, generator=g).cuda()
    by_expert = op(x, ids, w)
    op.by_expert_min_tokens = 10 ** 9
    per_pair = op(x, ids, w)
    assert rel(by_expert, per_pair) < 2e-6
    want = sum(w[:, j:j + 1].double() * torch.stack([(torch.nn.functional.silu(op.gate[e].double() @ x[t].double()) * (op.up[e].double() @ x[t].double())).to(dtype).double()
                                                   @ op.down[e].double().T for t, e in enumerate(ids[:, j].tolist())]) for j in range(top))
    assert rel(by_expert, want) < (1e-5 if dtype == torch.float32 else 2e-2)


def attention_alone(spec, dtype, n, page_size, portions, hs_scale_at=None, seed=4, width=24, hs_scale=12.0, tensor_path=True):
    """the operator over one sequence cut into `portions`, against the restatement over the whole sequence"""
    from ktransformers_b200.models.configuration_lekapel import LatentAttentionSpec
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.operators.attention import KLatentWindowAttention
    cfg = U.config([(spec, None)], width=width)
    W = {k[len("l0.mix."):]: v for k, v in U.weights(cfg, seed, dtype).items() if k.startswith("l0.mix.")}
    op = KLatentWindowAttention(width, LatentAttentionSpec.from_dict(spec), 1e-5, 0, dtype=dtype)
    op.load(DictLoader(W), "")
    op.use_tensor_path = tensor_path
    g = torch.Generator().manual_seed(seed)
    hs = torch.randn(n, width, generator=g)
    if hs_scale_at is not None:
        hs[hs_scale_at] *= hs_scale      # the un-normed rotated key part of this token grows: its scores stand out
    hs = hs.to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    past = (torch.zeros(0, spec["kv_rank"], dtype=torch.float64), torch.zeros(0, spec["rot_dim"], dtype=torch.float64), torch.zeros(0, dtype=torch.long))
    want, _ = O.latent_attention(hs.double(), torch.arange(n), past, Wd, spec, 1e-5)
    cache = PagedStateCache([spec["kv_rank"] + spec["rot_dim"]], width, n + page_size, 2, "cuda", dtype=dtype, page_size=page_size,
                            window=spec.get("mask", {}).get("size"))
    got, at = [], 0
    for p in portions:
        p = min(p, n - at)
        if p <= 0:
            break
        batch = cache.build_batch([("s", [0] * p, [])])
        got.append(op(hs[at:at + p].cuda().contiguous(), batch, cache))
        cache.commit()
        at += p
    assert at == n
    return torch.cat(got), want


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("spec", [U.mixer(), U.mixer(heads=9, dim=4, rot_dim=6, vdim=8, kv_rank=33, q_rank=8, window=None, rot_dims=2),
                                  U.mixer(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=64, q_rank=16, window=40, scale=0.3), U.mixer(window=1)])
def test_latent_window_attention_alone(dtype, tol, spec):
    got, want = attention_alone(spec, dtype, 70, 8, [70])
    assert rel(got, want) < tol
    got2, _ = attention_alone(spec, dtype, 70, 8, [33, 1, 1, 2, 30, 3])
    assert rel(got2, want) < tol


@gpu
@pytest.mark.parametrize("window", [5, 8, 17])
@pytest.mark.parametrize("decode", [False, True])
def test_window_edge_with_a_key_that_stands_out(window, decode):
    """token 20's key dominates: the rows that still see it (up to position 20 + window - 1) and the first that does not"""
    spec, spec_off = U.mixer(window=window, heads=4), U.mixer(window=window + 1, heads=4)
    n = 20 + window + 3
    inside, outside, bite = 20 + window - 1, 20 + window, 0.0
    for sign in (12.0, -12.0):           # the sign of a head's score for that key is random: one of the two makes it the largest
        got, want = attention_alone(spec, torch.float32, n, 4, [21] + [1] * n if decode else [n], hs_scale_at=20, hs_scale=sign)
        assert rel(got[inside], want[inside]) < 2e-5 and rel(got[outside], want[outside]) < 2e-5
        assert rel(got, want) < 2e-5
        _, shifted = attention_alone(spec_off, torch.float32, n, 4, [n], hs_scale_at=20, hs_scale=sign)
        bite = max(bite, rel(shifted[outside], want[outside]))
    assert bite > 1e-2                   # the test bites: seeing that one key a row too long moves the row far beyond the tolerance


@gpu
@pytest.mark.parametrize("heads,window,page", [(3, 40, 32), (70, None, 64), (64, 33, 32), (128, 150, 64)])
def test_tensor_core_path_at_latent_512_rot_64(heads, window, page):
    """kv_rank 512 / rot_dim 64 in bf16 takes the tcgen05 kernel: against the restatement, and against the CUDA-core kernel on
    the same bf16 inputs (what is left between the two is the order of the fp32 sums)"""
    spec = U.mixer(heads=heads, dim=16, rot_dim=64, vdim=8, kv_rank=512, q_rank=24, window=window)
    for portions, at in (([200], 7), ([129, 1, 1, 30, 2, 37], 100)):
        got, want = attention_alone(spec, torch.bfloat16, 200, page, portions, hs_scale_at=at)
        simple, _ = attention_alone(spec, torch.bfloat16, 200, page, portions, hs_scale_at=at, tensor_path=False)
        assert rel(got, want) < 4e-2 and rel(simple, want) < 4e-2
        assert rel(got, simple) < 1.5e-2


@gpu
def test_sink_counts_once_and_unscaled():
    spec = U.mixer(window=6, heads=2, scale=0.05)
    got, want = attention_alone(spec, torch.float32, 12, 4, [12], seed=9)
    assert rel(got, want) < 2e-5
    # with tiny scores the sink (weights ~ N(0,1), exp(sink) vs exp(~0) per key) takes a visible share: the first row sees one key
    from oracle.lekapel_oracle import sink_softmax_attention
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    o = sink_softmax_attention(q, torch.zeros(1, 1, 2, dtype=torch.float64), torch.ones(1, 1, 3, dtype=torch.float64), torch.tensor([0]), torch.tensor([0]), 1.0,
                               torch.tensor([0.0], dtype=torch.float64), None)
    assert abs(float(o[0, 0, 0]) - 0.5) < 1e-12


@gpu
def test_far_key_among_hundreds_split_path():
    """decode over a long un-windowed range takes the split kernel; a key far back stands out"""
    spec = U.mixer(window=None, heads=3, kv_rank=40)
    got, want = attention_alone(spec, torch.float32, 700, 16, [690] + [1] * 10, hs_scale_at=3)
    assert rel(got, want) < 2e-5
    spec = U.mixer(window=600, heads=3, kv_rank=40)
    got, want = attention_alone(spec, torch.float32, 700, 16, [690] + [1] * 10, hs_scale_at=95)     # 95 leaves the window at row 695
    assert rel(got, want) < 2e-5


# ------------------------------------------------------------------------------------------------ whole model (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_decode_and_portions_agree_with_the_restatement(tmp_path, dtype, tol):
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, dtype, max_tokens=128, max_slots=2, page_size=4)
    t = toks(75)                                                # the whole prompt takes the experts' grouped path, portions the per-pair one
    want = oracle_logits(om, t)
    err = rel if dtype == "float32" else rel_rows
    whole = run_steps(eng, cut("w", t, [75]))["w"]
    assert err(whole, want) < tol
    assert err(whole[:4], want[:4]) < tol                       # the first tokens of a sequence
    for sizes in ([1], [2], [3, 2, 7, 1, 5], [20, 2, 2, 1]):
        got = run_steps(eng, cut("p", t, sizes))["p"]
        assert err(got, want) < tol
        assert err(got, whole) < (1e-5 if dtype == "float32" else tol)   # the cut does not matter beyond rounding


@gpu
def test_other_sizes(tmp_path):
    for k, (layers, kw) in enumerate([
            ([(U.mixer(heads=1, dim=2, rot_dim=2, vdim=2, kv_rank=4, q_rank=2, window=2), U.moe(ff=3, experts=2, top=2))], dict(width=8, groups=1, residual_mult=1.0, logit_scale=1.0)),
            ([(U.mixer(heads=16, dim=12, rot_dim=8, vdim=10, kv_rank=96, q_rank=48, window=9, rot_dims=6), U.dense(100)), (U.mixer(window=3), None)] * 2,
             dict(width=72, groups=6, vocab=31)),
            ([(U.mixer(heads=5, kv_rank=130, window=11), U.moe(ff=20, experts=9, top=3)), (U.mixer(window=None), U.dense(8))], dict(width=40, groups=2))]):
        cfg = U.config(layers, **kw)
        eng, om = serve(tmp_path, cfg, "float32", seed=10 + k, max_tokens=64, max_slots=2, page_size=8)
        t = toks(30, cfg["vocab"], seed=k)
        assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], oracle_logits(om, t)) < F32_TOL


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations(tmp_path, seed):
    """sizes, layer order and constants drawn per seed (odd sizes, head counts that are no multiple of 8, windows around 32 and
    64, experts with top from 1 to all): one prompt whole, in uneven portions, and with a decoded tail"""
    import random
    r = random.Random(seed)
    width = r.choice([16, 40, 136, 320])
    layers = []
    for _ in range(r.randint(1, 4)):
        rot_dim = r.choice([2, 6, 8, 16, 32])
        m = U.mixer(heads=r.choice([1, 2, 5, 8, 12, 20]), dim=r.choice([4, 7, 24, 64]), rot_dim=rot_dim, vdim=r.choice([5, 8, 48]),
                    kv_rank=r.choice([8, 33, 130, 256]), q_rank=r.choice([8, 12, 80]), window=r.choice([1, 2, 9, 31, 32, 33, 64, 65, None]),
                    base=r.choice([100.0, 5e5]), rot_dims=r.choice([rot_dim, max(2, rot_dim // 4 * 2)]), scale=r.choice([None, 0.125]))
        e = r.choice([2, 3, 17, 32])
        layers.append((m, r.choice([None, U.dense(ff=r.choice([8, 100, 1030])), U.moe(ff=r.choice([4, 12, 96]), experts=e, top=r.randint(1, min(e, 8)))])))
    cfg = U.config(layers, vocab=r.choice([31, 77, 1000]), width=width, groups=r.choice([1, 2, 4, 8]), eps=r.choice([1e-5, 1e-3]),
                   residual_mult=r.choice([1.0, 0.3]), logit_scale=r.choice([1.0, 2.0]))
    eng, om = serve(tmp_path, cfg, "float32", seed=seed, max_tokens=256, max_slots=2, page_size=r.choice([4, 16, 64]))
    t = toks(r.choice([40, 90, 150]), cfg["vocab"], seed=seed)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([len(t)], [3, 17, 2, 1, 33, 2, 64], [len(t) - 20] + [1] * 20)):
        assert rel(run_steps(eng, cut(("d", k), t, sizes))[("d", k)], want) < F32_TOL


@gpu
def test_captured_decode_steps_with_a_key_range_cut_for_a_large_cache(tmp_path):
    """a roomy cache makes the replayed decode step cut its key range into many parts, most of them empty for a short sequence"""
    cfg = U.config([(U.mixer(window=None, heads=3), U.moe()), (U.mixer(window=300, heads=2, kv_rank=40), U.dense(16))])
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=8192, max_slots=2, page_size=16)
    for r, n in enumerate((40, 330)):
        t = toks(n, seed=40 + r)
        got = run_steps(eng, cut(("g", r), t, [n - 12] + [1] * 12))[("g", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
    assert 1 in eng._captured and eng._captured[1].graph is not None


@gpu
def test_long_expert_rows_decode_without_capture(tmp_path):
    """expert rows beyond the small-batch kernels' shared memory: decode takes the grouped path, which reads the routing counts
    on the host in fp32, so the engine does not replay such a model's decode steps as graphs; the results still agree"""
    cfg = U.config([(U.mixer(), U.moe(ff=13000, experts=5, top=5))], width=16, groups=2)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=64, max_slots=2)
    assert not eng.model.decode_is_capturable() and not eng.cuda_graphs
    t = toks(14, seed=5)
    got = run_steps(eng, cut("x", t, [6] + [1] * 8))["x"]
    assert rel(got, oracle_logits(om, t)) < F32_TOL
    assert not eng._captured


@gpu
def test_unequal_requests_in_one_batch_equal_each_alone(tmp_path):
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=256, max_slots=4, page_size=4)
    ta, tb, tc = toks(23, seed=1), toks(9, seed=2), toks(14, seed=3)
    steps = [[("a", ta[:10], False), ("b", tb[:1], False)],
             [("a", ta[10:11], False), ("b", tb[1:9], True), ("c", tc[:2], False)],
             [("c", tc[2:14], True), ("a", ta[11:23], True)]]
    got = run_steps(eng, steps)
    for i, t in (("a", ta), ("b", tb), ("c", tc)):
        assert rel(got[i], oracle_logits(om, t)) < F32_TOL
        alone = run_steps(eng, cut(i + "'", t, [len(t)]))[i + "'"]
        assert rel(got[i], alone) < 1e-5


@gpu
def test_long_decode_over_reused_pages_and_slots(tmp_path):
    """window 5 / 7 and pages of 4: a long decode walks over pages that were given back; sequences come and go in 2 slots"""
    cfg = U.config(MIXED[:2])
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=40, max_slots=2, page_size=4)
    assert eng.cache.window == 7
    for r in range(3):
        t = toks(90, seed=20 + r)
        got = run_steps(eng, cut(("s", r), t, [6] + [1] * 84))[("s", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
        short = toks(3, seed=30 + r)
        assert rel(run_steps(eng, cut(("t", r), short, [3]))[("t", r)], oracle_logits(om, short)) < F32_TOL
    assert len(eng.cache._free_pages) == eng.cache.num_pages and len(eng.cache._free_slots) == 2


@gpu
def test_greedy_generation_through_the_scheduler_and_the_command_line(tmp_path, capsys):
    from ktransformers_b200 import local_chat
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=256, max_slots=3, page_size=4, max_step_tokens=7)
    prompts = [toks(12, seed=5), toks(3, seed=6), toks(20, seed=7), toks(1, seed=8)]
    want = []
    for p in prompts:
        st, out = om.new_state(), []
        nxt = int(om.forward(p, st)[-1].argmax())
        for _ in range(6):
            out.append(nxt)
            nxt = int(om.forward([nxt], st)[-1].argmax())
        want.append(out)
    assert eng.generate(prompts, 6) == want                      # 4 requests, 3 slots, 7 tokens per step: portions and decode mix
    assert len(eng.cache._free_slots) == 3
    args = ["--model_path", str(tmp_path / "ckpt0"), "--dtype", "float32", "--max_new_tokens", "6", "--chunk_size", "5"]
    for p in prompts[:2]:
        args += ["--prompt_ids", ",".join(map(str, p))]
    assert local_chat.main(args) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines() if l.startswith("{")]
    assert [l["output"] for l in lines] == want[:2]


@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_trace_replay_runner(tmp_path, dtype, tol):
    """bin/trace_run as a process: steps on standard input, one logits file per step that asks for some, `done <n>` lines"""
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = U.config(MIXED[:2], vocab=41)
    w = U.weights(cfg, 5, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / "m", cfg, w)
    om = O.Model(cfg, w, torch.float64)
    a, b = toks(21, 41, seed=1), toks(9, 41, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[15:17], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[17:18], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[18:21], "want": [2, 1]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    la, lb = oracle_logits(om, a), oracle_logits(om, b)
    want = {0: la[[0, 14]], 2: la[[17]], 3: la[[20, 19]], 4: lb[[8]]}
    assert not (out / "1.f32").exists()
    err = rel if dtype == "float32" else rel_rows
    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 41))
        assert got.shape == ref.shape and err(got, ref) < tol
