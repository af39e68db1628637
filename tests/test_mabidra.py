"""Mabidra through the framework (registry, loader, paged state cache, scheduler, engine, CUDA operators) against the plain
restatement in oracle/mabidra_oracle.py, on small random checkpoints made here.  CPU tests cover the host logic."""
import json
import random

import pytest
import torch

import mabidra_util as U
from oracle import mabidra_oracle as O

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


MIXED = [(U.attn(), U.dense()), (U.gla(), U.moe()), (U.attn(heads=6, kv_heads=6, dim=5, vdim=3, rows=6, bias_max=9.5, every=5), None),
         (U.gla(heads=2, dim=17, vdim=33, tau=9.0, rank=3), U.moe(ff=8, experts=3, top=1))]
LOOP = (1, 3, 2)


def serve(tmp_path, cfg, dtype, seed=0, **engine_kw):
    from ktransformers_b200.models import load_model
    from ktransformers_b200.util.engine import Engine
    w = U.weights(cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / f"ckpt{seed}", cfg, w)
    torch.backends.cuda.matmul.allow_tf32 = False
    model = load_model(path, dtype)
    return Engine(model, **engine_kw), O.Model(cfg[0], w, torch.float64)


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
def test_config_reads_sizes_per_layer_and_lays_out_the_runs():
    from ktransformers_b200.models.configuration_mabidra import MabidraConfig
    c = MabidraConfig.from_dict(U.config(MIXED, vocab=77, width=36, groups=2, emb_scale=0.25, loop=LOOP)[0])
    assert (c.vocab, c.width, c.norm_groups, c.embedding_scale, len(c.layers)) == (77, 36, 2, 0.25, 4)
    assert c.layers[0].mixer.kv_heads == 2 and c.layers[2].mixer.kv_heads == 6 and c.layers[2].mixer.bias_max == 9.5 and c.layers[2].mixer.temp_every == 5
    assert c.layers[1].mixer.tau == 4.0 and c.layers[3].mixer.vdim == 33 and c.layers[2].mlp is None and c.layers[3].mlp.top == 1
    assert c.layer_runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]          # the pass number stands at the run that opens it
    assert c.cache_row_widths() == [2 * 16, 0, 6 * 8, 0, 6 * 8, 0] and c.state_widths() == [0, 210, 0, 210, 0, 2 * 17 * 33]
    assert c.num_hidden_layers == 6 and c.max_window() is None
    plain = MabidraConfig.from_dict(U.config(MIXED)[0])
    assert plain.loop is None and plain.layer_runs() == [(i, None) for i in range(4)]
    whole = MabidraConfig.from_dict(U.config(MIXED, loop=(0, 4, 3))[0])
    assert whole.layer_runs()[:5] == [(0, 0), (1, None), (2, None), (3, None), (0, 1)] and whole.num_hidden_layers == 12
    with pytest.raises(ValueError):
        MabidraConfig.from_dict(U.config(MIXED, loop=(2, 5, 2))[0])


def test_registry_picks_the_class_by_config():
    from ktransformers_b200.models import architecture_of, model_class
    assert model_class(architecture_of({"architecture": "Mabidra"})).__name__ == "MabidraForCausalLM"


@pytest.mark.parametrize("rows,reach", [(8, 11), (6, 9.5), (24, 200), (2, 5), (16, 8.5), (12, 1000)])
def test_distance_bias_table_lists_the_bucket_of_every_distance(rows, reach):
    from ktransformers_b200.operators.attention import distance_bias_table
    rel_t = torch.arange(rows * 3, dtype=torch.float32).reshape(rows, 3)
    table = distance_bias_table(rel_t, reach)
    n = table.shape[1]                                           # [heads, distances]
    assert table.shape[0] == 3 and n <= int(reach) + 2 and O.distance_bucket(n - 1, rows, reach) == rows - 1
    for dist in list(range(n + 5)) + [10 ** 6]:
        assert torch.equal(table[:, min(dist, n - 1)], rel_t[O.distance_bucket(dist, rows, reach)])
    assert [O.distance_bucket(x, 8, 11) for x in (0, 3, 4, 5, 10, 11, 12)] == [0, 3, 4, 4, 7, 7, 7]


def test_oracle_portions_equal_whole_prompt_and_both_attention_forms_agree():
    cfg = U.config(MIXED, loop=LOOP)
    w = U.weights(cfg, 3, torch.float32)
    om = O.Model(cfg[0], w, torch.float64)
    t = toks(19)
    whole = oracle_logits(om, t)
    st, parts = om.new_state(), []
    for lo, hi in ((0, 1), (1, 3), (3, 10), (10, 11), (11, 19)):
        parts.append(om.forward(t[lo:hi], st).float())
    assert rel(torch.cat(parts), whole) < 1e-6
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(5, 4, 3, generator=g).double(), torch.randn(9, 2, 3, generator=g).double(), torch.randn(9, 2, 2, generator=g).double()
    args = (q, k, v, torch.arange(4, 9), torch.arange(9), 0.3, torch.randn(6, 4, generator=g).double(), torch.randn(4, generator=g).double(), 7.5)
    assert rel(O.sigmoid_attention_fast(*args), O.sigmoid_attention(*args)) < 1e-12
    assert float(O.xielu(torch.tensor(0.0).double(), torch.tensor(0.3), torch.tensor(-0.2))) == 0.0


def test_batch_lists_state_rows_per_sequence_portion():
    from ktransformers_b200.models.custom_cache import PagedStateCache
    c = PagedStateCache([6, 0], [0, 12], max_tokens=32, max_slots=2, device="cpu", dtype=torch.float32, page_size=4)
    assert c.state[0].shape == (4, 0) and c.state[1].shape == (4, 12) and c.key_cache[1].shape[-1] == 0
    b = c.build_batch([("a", [1, 2, 3], [2]), ("b", [7], [0])])
    assert b.n_seqs == 2 and b.seqs[:, :2].tolist() == [[0, 3], [3, 1], [-1, -1], [1, 3]]          # first row, count, read row, write row
    c.commit()
    b = c.build_batch([("b", [9, 9], []), ("a", [4], [0])])
    assert b.seqs[:, :2].tolist() == [[0, 2], [2, 1], [3, 1], [2, 0]]
    c.commit()
    c.close("a")
    b = c.build_batch([("c", [5], [])])
    assert b.slot.tolist() == [0] and b.seqs[:, :1].tolist() == [[0], [1], [-1], [1]]              # a reused slot starts without state


# ------------------------------------------------------------------------------------------------ mechanisms alone (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("groups,width", [(1, 20), (3, 36), (4, 256), (5, 35), (2, 6), (2, 512), (8, 64), (1, 1024)])      # one group after the other / all groups together
def test_sandwich_norm_kernel(dtype, tol, groups, width):
    from ktransformers_b200.operators.norm import KGroupRMSNorm
    g = torch.Generator().manual_seed(1)
    x, y, row = torch.randn(7, width, generator=g), torch.randn(7, width, generator=g) * 3, torch.randn(width, generator=g)
    post, pre = (KGroupRMSNorm(width, groups, 1e-4, dtype=dtype) for _ in range(2))
    for n in (post, pre):
        n.load(DictLoader({"w": (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)}), "w")
    wp, wq = post.weight.double().cpu(), pre.weight.double().cpu()
    for y_dt in (dtype, torch.float32):
        yd = y.to(y_dt)
        want_x = x.double() + O.grouped_rms_norm(yd.double(), wp, groups, 1e-4)
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, pre)
        assert rel(xo, want_x) < 1e-6 and rel(h, O.grouped_rms_norm(want_x, wq, groups, 1e-4)) < tol
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, None)
        assert h is None and rel(xo, want_x) < 1e-6
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, pre, keep_x=False)
        assert xo is None and rel(h, O.grouped_rms_norm(want_x, wq, groups, 1e-4)) < tol
        xo, h = KGroupRMSNorm.fused(None, yd.cuda(), None, pre, row_add=row.cuda())       # the stream restarts from y plus a row
        assert rel(xo, yd.double() + row.double()) < 1e-6 and rel(h, O.grouped_rms_norm(yd.double() + row.double(), wq, groups, 1e-4)) < tol


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_xielu_mlp(dtype, tol):
    from ktransformers_b200.operators.mlp import KXIELUMLP
    g = torch.Generator().manual_seed(2)
    for pq in ([0.7, -0.4], [-3.0, 2.5]):
        up, down, act = (torch.randn(52, 24, generator=g) * 0.6).to(dtype), torch.randn(24, 52, generator=g).to(dtype), torch.tensor(pq).to(dtype)
        op = KXIELUMLP(24, 52, dtype=dtype)
        op.load(DictLoader({"up": up, "down": down, "act": act}), "")
        h = (torch.randn(9, 24, generator=g) * 2).to(dtype)
        assert rel(op(h.cuda()), O.xielu_mlp(h.double(), up.double(), down.double(), act.double())) < tol
    z = torch.tensor([[-30.0, -1.0, -1e-4, 0.0, 1e-4, 2.0, 30.0]])
    from ktransformers_b200 import native
    out = torch.empty_like(z).cuda()
    native.check_seq(native.seq_lib().ktb200_xielu(z.cuda().data_ptr(), out.data_ptr(), op.pq.data_ptr(), z.numel(), native.GGML_F32, torch.cuda.current_stream().cuda_stream))
    assert rel(out, O.xielu(z.double(), op.pq[0].double().cpu(), op.pq[1].double().cpu())) < 1e-6


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("experts,top,ff,width", [(5, 2, 12, 24), (3, 1, 7, 20), (16, 4, 64, 128), (4, 4, 6, 18), (2, 1, 33, 9)])
@pytest.mark.parametrize("tokens", [1, 11, 70])              # an expert's rows once for several pairs / grouped GEMMs
def test_topk_softmax_moe_with_relu_squared_experts(dtype, tol, experts, top, ff, width, tokens):
    from ktransformers_b200.operators.experts import KTopKSoftmaxMoE
    g = torch.Generator().manual_seed(3)
    W = {"router": (torch.randn(experts, width, generator=g) * 0.5).to(dtype), "router.b": (torch.randn(experts, generator=g) * 2).to(dtype)}
    for e in range(experts):
        W[f"e{e}.up"], W[f"e{e}.down"] = ((torch.randn(s, generator=g) * 0.3).to(dtype) for s in ((ff, width), (width, ff)))
    op = KTopKSoftmaxMoE(width, ff, experts, top, dtype=dtype)
    op.load(DictLoader(W), "")
    h = torch.randn(tokens, width, generator=g).to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    ids, w = op.router(h.cuda())
    oi, ow = O.topk_softmax_router(h.double(), Wd["router"], Wd["router.b"], top)
    assert torch.equal(ids.cpu().sort(-1).values, oi.sort(-1).values)
    assert rel(w.cpu().sort(-1).values, ow.sort(-1).values) < 1e-5 and rel(w.sum(-1), torch.ones(tokens)) < 1e-5     # one chosen expert weighs 1
    assert rel(op(h.cuda()), O.relu2_moe_mlp(h.double(), Wd, top)) < tol
    op.experts.by_expert_min_tokens = 10 ** 9                   # the per-pair kernels
    assert rel(op(h.cuda()), O.relu2_moe_mlp(h.double(), Wd, top)) < tol


def mixer_alone(desc, dtype, n, page_size, portions, big_at=None, big=30.0, seed=4, width=24, tweak=None, tensor_cores=True):
    """one mixer operator over one sequence cut into `portions`, against the restatement over the whole sequence; `big_at`:
    the input row of that token is scaled, so its un-normed value (and key, for the recurrence) stands out"""
    from ktransformers_b200.models.configuration_mabidra import MIXER_SPECS
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.models.modeling_mabidra import MIXERS
    cfg = U.config([(desc, None)], width=width)
    W = {k[len("l0.mix."):]: v for k, v in U.weights(cfg, seed, dtype).items() if k.startswith("l0.mix.")}
    if tweak:
        tweak(W)
    m = desc["mixer"]
    spec = MIXER_SPECS[desc["type"]].from_dict(m)
    op = MIXERS[desc["type"]](width, spec, 1e-5, dtype=dtype)
    op.load(DictLoader(W), "")
    op.use_tensor_cores = tensor_cores
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(n, width, generator=g)
    if big_at is not None:
        h[big_at] *= big
    h = h.to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    if desc["type"] == "attention":
        past = (torch.zeros(0, m["kv_heads"], m["dim"], dtype=torch.float64), torch.zeros(0, m["kv_heads"], m["vdim"], dtype=torch.float64), torch.zeros(0, dtype=torch.long))
        want, _ = O.attention_mixer(h.double(), torch.arange(n), past, Wd, m, 1e-5)
    else:
        want, _ = O.gla_mixer(h.double(), torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=torch.float64), Wd, m, 1e-5)
    cache = PagedStateCache([spec.cache_row_width()], [spec.state_width()], n + page_size, 2, "cuda", dtype=dtype, page_size=page_size)
    got, at, k = [], 0, 0
    while at < n:                                                # the last size repeats
        p = min(portions[min(k, len(portions) - 1)], n - at)
        batch = cache.build_batch([("s", [0] * p, [])])
        got.append(op(h[at:at + p].cuda().contiguous(), batch, cache, 0))
        cache.commit()
        at, k = at + p, k + 1
    return torch.cat(got), want


ATTN_SHAPES = [U.attn(), U.attn(heads=6, kv_heads=6, dim=5, vdim=3, rows=6, bias_max=9.5, every=5), U.attn(heads=9, kv_heads=1, dim=16, vdim=40, rows=24, bias_max=60, every=50),
               U.attn(heads=20, kv_heads=2, dim=7, vdim=70, rows=2, bias_max=3, coef=0.0), U.attn(heads=1, kv_heads=1, dim=33, vdim=1, scale=0.9, rows=10, bias_max=500, every=1)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("desc", ATTN_SHAPES)
def test_sigmoid_attention_alone(dtype, tol, desc):
    got, want = mixer_alone(desc, dtype, 70, 8, [70])
    assert rel(got, want) < tol
    assert rel(got[:3], want[:3]) < tol                          # the first tokens: one, two, three visible keys
    got2, _ = mixer_alone(desc, dtype, 70, 8, [33, 1, 1, 2, 30, 3])
    assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)


@gpu
@pytest.mark.parametrize("rows,reach", [(8, 11), (6, 9.5), (16, 40)])
@pytest.mark.parametrize("decode", [False, True])
def test_distance_bucket_edges_with_a_value_that_stands_out(rows, reach, decode):
    """token 20's value dominates every later row, weighted by the bias of its distance: the rows just before and after every
    change of bucket, around the table's reach and far beyond it.  A table that reaches further must differ."""
    spread = lambda W: W.__setitem__("rel", torch.linspace(-4, 4, rows)[:, None].repeat(1, W["rel"].shape[1]) * torch.tensor([1.0, -1.0, 0.5, 2.0])[:W["rel"].shape[1]])
    desc, other = U.attn(rows=rows, bias_max=reach), U.attn(rows=rows, bias_max=reach * 1.6)
    n = 20 + int(reach) + 40
    got, want = mixer_alone(desc, torch.float32, n, 4, [21] + [1] * n if decode else [n], big_at=20, tweak=spread)
    assert rel(got, want) < 2e-5
    edges = [d for d in range(1, int(reach) + 3) if O.distance_bucket(d, rows, reach) != O.distance_bucket(d - 1, rows, reach)]
    assert len(edges) >= rows - 2
    for d in edges + [int(reach) + 30]:
        assert rel(got[20 + d - 1], want[20 + d - 1]) < 2e-5 and rel(got[20 + d], want[20 + d]) < 2e-5
    _, shifted = mixer_alone(other, torch.float32, n, 4, [n], big_at=20, tweak=spread)
    assert max(rel(shifted[20 + d], want[20 + d]) for d in range(1, int(reach) + 3)) > 1e-2          # the test bites


@gpu
def test_far_value_among_hundreds_and_the_split_path():
    """decode over a long range cuts the keys into parts; a value far back stands out, and so does one at a part's edge"""
    for at in (3, 127, 128, 383, 384):
        got, want = mixer_alone(U.attn(heads=3, kv_heads=1, dim=12, vdim=9), torch.float32, 700, 16, [690] + [1] * 10, big_at=at)
        assert rel(got, want) < 2e-5
    got, want = mixer_alone(U.attn(heads=16, kv_heads=2), torch.bfloat16, 600, 64, [590, 2] + [1] * 8, big_at=64)
    assert rel(got, want) < 4e-2


MMA_SHAPES = [U.attn(heads=8, kv_heads=2, dim=16, vdim=32), U.attn(heads=9, kv_heads=1, dim=48, vdim=16, rows=24, bias_max=60, every=50),
              U.attn(heads=34, kv_heads=2, dim=32, vdim=32, rows=6, bias_max=9.5), U.attn(heads=4, kv_heads=4, dim=128, vdim=128, rows=16, bias_max=100, every=50),
              U.attn(heads=12, kv_heads=1, dim=64, vdim=80, rows=4, bias_max=300), U.attn(heads=40, kv_heads=2, dim=16, vdim=112, rows=8, bias_max=70)]


@gpu
@pytest.mark.parametrize("desc", MMA_SHAPES)
def test_tensor_core_attention_path(desc):
    """bf16 with head sizes that are multiples of 16 takes the tensor-core tiles: against the restatement, and against the
    CUDA-core kernel on the same bf16 inputs (between the two: bf16 weights in the second product, and the order of the sums).
    200 tokens cross three key tiles; portions start and end inside tiles; the value that stands out sits at a tile's edge"""
    for portions, at in (([200], 7), ([129, 1, 1, 30, 2, 37], 63), ([64, 64, 8, 1], 64), ([190] + [1] * 10, 127)):
        got, want = mixer_alone(desc, torch.bfloat16, 200, 16, portions, big_at=at)
        simple, _ = mixer_alone(desc, torch.bfloat16, 200, 16, portions, big_at=at, tensor_cores=False)
        assert rel(got, want) < 4e-2 and rel(simple, want) < 4e-2
        assert rel(got, simple) < 1.5e-2
        assert rel(got[:3], want[:3]) < 4e-2 and rel(got[at:at + 3], want[at:at + 3]) < 4e-2


@gpu
def test_tensor_core_attention_far_value_and_split_edges():
    """decode over a long range on the tensor-core path cuts the keys into parts of whole tiles"""
    desc = U.attn(heads=16, kv_heads=2, dim=32, vdim=48)
    for at in (3, 127, 128, 383, 384, 640):
        got, want = mixer_alone(desc, torch.bfloat16, 700, 64, [690] + [1] * 10, big_at=at)
        simple, _ = mixer_alone(desc, torch.bfloat16, 700, 64, [690] + [1] * 10, big_at=at, tensor_cores=False)
        assert rel(got, want) < 4e-2 and rel(got[690:], want[690:]) < 4e-2 and rel(got, simple) < 1.5e-2


@gpu
def test_bias_table_too_long_for_shared_memory():
    """a table that reaches 5000 tokens is read from global memory by the CUDA-core kernel; the value that stands out sits inside
    and outside the logarithmic part"""
    desc = U.attn(heads=8, kv_heads=1, dim=8, vdim=8, rows=16, bias_max=5000)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 4e-2)):
        got, want = mixer_alone(desc, dtype, 300, 64, [290] + [1] * 10, big_at=5)
        assert rel(got, want) < tol


GLA_SHAPES = [U.gla(), U.gla(heads=2, dim=17, vdim=33, tau=9.0, rank=3), U.gla(heads=1, dim=64, vdim=64, tau=12.0, rank=8), U.gla(heads=5, dim=3, vdim=1, tau=1.0, rank=1),
              U.gla(heads=2, dim=130, vdim=70, tau=30.0, rank=4)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("desc", GLA_SHAPES)
def test_gated_linear_attention_alone(dtype, tol, desc):
    got, want = mixer_alone(desc, dtype, 70, 8, [70])
    assert rel(got, want) < tol and rel(got[:3], want[:3]) < tol
    for portions in ([33, 1, 1, 2, 30, 3], [2], [15, 1, 16, 17, 1], [1]):      # the kernel stages 16 tokens at a time: portions that end on, before and after that edge
        got2, _ = mixer_alone(desc, dtype, 70, 8, portions)
        assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)


@gpu
@pytest.mark.parametrize("decode", [False, True])
def test_recurrent_state_carries_a_far_token(decode):
    """slow decay (sigmoid(z + 6)^(1/50) per token): the key and value of token 5, scaled up, still dominate 300 tokens later; a
    state that were lost or reset on the way would show at once"""
    slow = lambda W: W.__setitem__("a2.b", W["a2.b"] + 6.0)
    desc = U.gla(heads=2, dim=12, vdim=9, tau=50.0)
    got, want = mixer_alone(desc, torch.float32, 320, 8, [200] + [1] * 120 if decode else [7, 100, 2, 211], big_at=5, tweak=slow)
    assert rel(got, want) < 3e-5 and rel(got[300:], want[300:]) < 3e-5
    plain, _ = mixer_alone(desc, torch.float32, 320, 8, [320], tweak=slow)
    assert rel(plain[300:], want[300:]) > 1e-1                   # the test bites: without the far token the late rows differ


# ------------------------------------------------------------------------------------------------ whole model (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_decode_and_portions_agree_with_the_restatement(tmp_path, dtype, tol):
    cfg = U.config(MIXED, loop=LOOP)
    eng, om = serve(tmp_path, cfg, dtype, max_tokens=128, max_slots=2, page_size=4)
    t = toks(75)                                                # the whole prompt takes the experts' grouped path, portions the small-batch one
    want = oracle_logits(om, t)
    err = rel if dtype == "float32" else rel_rows
    whole = run_steps(eng, cut("w", t, [75]))["w"]
    assert err(whole, want) < tol
    assert err(whole[:4], want[:4]) < tol                       # the first tokens of a sequence
    for sizes in ([1], [2], [3, 2, 7, 1, 5], [20, 2, 2, 1]):
        got = run_steps(eng, cut("p", t, sizes))["p"]
        assert err(got, want) < tol
        assert err(got, whole) < (2e-5 if dtype == "float32" else tol)   # the cut does not matter beyond rounding


@gpu
def test_whole_model_in_bf16_on_tensor_core_head_sizes(tmp_path):
    """head sizes that are multiples of 16: bf16 attention runs on the tensor-core tiles inside a whole model (a looped span,
    grouped heads, 150 tokens over three key tiles), whole, in portions and with a decoded tail"""
    layers = [(U.attn(heads=6, kv_heads=2, dim=32, vdim=48, rows=12, bias_max=40, every=20), U.dense(96)), (U.gla(heads=4, dim=32, vdim=16, tau=6.0), U.moe(ff=32, experts=6, top=2)),
              (U.attn(heads=4, kv_heads=4, dim=16, vdim=16, rows=6, bias_max=100), U.moe(ff=16, experts=4, top=1))]
    cfg = U.config(layers, width=64, groups=2, vocab=90, loop=(1, 3, 2))
    eng, om = serve(tmp_path, cfg, "bfloat16", seed=3, max_tokens=512, max_slots=2, page_size=16)
    t = toks(150, 90, seed=9)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([150], [70, 3, 2, 40, 1, 34], [130] + [1] * 20)):
        assert rel_rows(run_steps(eng, cut(("m", k), t, sizes))[("m", k)], want) < BF16_TOL


def test_distance_table_refuses_a_reach_inside_the_exact_part():
    from ktransformers_b200.operators.attention import distance_bias_table
    with pytest.raises(ValueError):
        distance_bias_table(torch.zeros(8, 2), 4.0)


@gpu
def test_residual_stream_after_every_layer_run(tmp_path):
    cfg = U.config(MIXED, loop=LOOP)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=64, max_slots=2, page_size=8)
    t = toks(11, seed=2)
    want, got = [], []
    om.forward(t, om.new_state(), want)
    eng.model(eng.cache.build_batch([("r", t, [])]), eng.cache, got)
    assert len(got) == len(want) == 6
    for a, b in zip(got, want):
        assert rel(a, b) < 1e-4


@gpu
def test_other_sizes_and_layer_orders(tmp_path):
    cases = [
        ([(U.gla(heads=1, dim=2, vdim=2, tau=1.5, rank=1), U.moe(ff=3, experts=2, top=2))], dict(width=8, groups=1, emb_scale=1.0)),                                 # no loop, one layer
        ([(U.attn(heads=16, kv_heads=4, dim=12, vdim=10, rows=12, bias_max=30), U.dense(100)), (U.gla(), None)] * 2, dict(width=72, groups=6, vocab=31, loop=(0, 4, 3))),   # everything loops
        ([(U.gla(heads=5, dim=24, vdim=24), U.moe(ff=20, experts=9, top=9)), (U.attn(heads=2, kv_heads=1, dim=8, vdim=8), U.dense(8)), (U.attn(), U.moe(top=1))],
         dict(width=40, groups=2, loop=(2, 3, 1))),                                                                                                              # one pass over the last layer
        ([(U.attn(), None), (U.attn(rows=4, bias_max=2.5), U.dense(16)), (U.gla(), U.dense(24))], dict(width=16, groups=4, loop=(0, 2, 2), eps=1e-3))]
    for k, (layers, kw) in enumerate(cases):
        cfg = U.config(layers, **kw)
        eng, om = serve(tmp_path, cfg, "float32", seed=10 + k, max_tokens=64, max_slots=2, page_size=8)
        t = toks(30, cfg[0]["vocab"], seed=k)
        assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], oracle_logits(om, t)) < F32_TOL


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations(tmp_path, seed):
    """sizes, layer order, loop and constants drawn per seed: one prompt whole, in uneven portions, and with a decoded tail"""
    r = random.Random(seed)
    width = r.choice([16, 40, 136, 320])
    layers = []
    for _ in range(r.randint(1, 5)):
        if r.random() < 0.5:
            G = r.choice([1, 2, 3, 4])
            rows = r.choice([2, 6, 8, 16, 24])
            m = U.attn(heads=G * r.choice([1, 2, 5, 9]), kv_heads=G, dim=r.choice([4, 7, 24, 64]), vdim=r.choice([5, 8, 48, 96]), scale=r.choice([None, 0.11]),
                       bias_max=rows // 2 + r.choice([1.5, 7, 40, 300]), rows=rows, coef=r.choice([0.0, 0.25, 1.0]), every=r.choice([1, 4, 32, 1000]))
        else:
            m = U.gla(heads=r.choice([1, 2, 5, 8]), dim=r.choice([4, 7, 24, 64, 100]), vdim=r.choice([5, 8, 32, 48, 65]), tau=r.choice([1.0, 7.5, 20.0]), rank=r.choice([1, 4, 16]))
        e = r.choice([2, 3, 17, 32])
        layers.append((m, r.choice([None, U.dense(ff=r.choice([8, 100, 1030])), U.moe(ff=r.choice([4, 12, 96]), experts=e, top=r.randint(1, min(e, 8)))])))
    loop = None
    if r.random() < 0.75:
        a = r.randrange(len(layers))
        loop = (a, r.randint(a + 1, len(layers)), r.randint(1, 3))
    cfg = U.config(layers, vocab=r.choice([31, 77, 1000]), width=width, groups=r.choice([1, 2, 4, 8]), eps=r.choice([1e-5, 1e-3]), emb_scale=r.choice([1.0, 0.3, 4.0]), loop=loop)
    eng, om = serve(tmp_path, cfg, "float32", seed=seed, max_tokens=256, max_slots=2, page_size=r.choice([4, 16, 64]))
    t = toks(r.choice([40, 90, 150]), cfg[0]["vocab"], seed=seed)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([len(t)], [3, 17, 2, 1, 33, 2, 64], [len(t) - 20] + [1] * 20)):
        assert rel(run_steps(eng, cut(("d", k), t, sizes))[("d", k)], want) < F32_TOL


@gpu
def test_captured_decode_steps_with_a_key_range_cut_for_a_large_cache(tmp_path):
    """a roomy cache makes the replayed decode step cut its key range into many parts, most of them empty for a short sequence;
    the recurrent state rows flip between the replays"""
    cfg = U.config(MIXED, loop=LOOP)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=8192, max_slots=2, page_size=16)
    for r, n in enumerate((40, 330)):
        t = toks(n, seed=40 + r)
        got = run_steps(eng, cut(("g", r), t, [n - 12] + [1] * 12))[("g", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
    assert 1 in eng._captured and eng._captured[1].graph is not None


@gpu
def test_unequal_requests_in_one_batch_equal_each_alone(tmp_path):
    cfg = U.config(MIXED, loop=LOOP)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=256, max_slots=4, page_size=4)
    ta, tb, tc = toks(23, seed=1), toks(9, seed=2), toks(14, seed=3)
    steps = [[("a", ta[:10], False), ("b", tb[:1], False)],
             [("a", ta[10:11], False), ("b", tb[1:9], True), ("c", tc[:2], False)],
             [("c", tc[2:14], True), ("a", ta[11:23], True)]]
    got = run_steps(eng, steps)
    for i, t in (("a", ta), ("b", tb), ("c", tc)):
        assert rel(got[i], oracle_logits(om, t)) < F32_TOL
        alone = run_steps(eng, cut(i + "'", t, [len(t)]))[i + "'"]
        assert rel(got[i], alone) < 2e-5


@gpu
def test_long_decode_over_reused_pages_and_slots(tmp_path):
    """pages of 4 and 2 slots: sequences come and go, pages and state rows are handed out again un-cleared, and a new sequence in
    a used slot must start from an empty state"""
    cfg = U.config(MIXED[:2] + [(U.gla(heads=2, dim=8, vdim=8, tau=40.0), None)], loop=(1, 3, 2))
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=120, max_slots=2, page_size=4)
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
    cfg = U.config(MIXED, loop=LOOP)
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
    cfg = U.config(MIXED[:2], vocab=41, loop=(1, 2, 2))
    w = U.weights(cfg, 5, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / "m", cfg, w)
    om = O.Model(cfg[0], w, torch.float64)
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
