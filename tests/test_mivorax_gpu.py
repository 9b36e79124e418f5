"""Mivorax on the GPU against the plain implementation (tests/plain_mivorax.py): every mechanism alone, prompts
against token-by-token decoding, portions down to two tokens, unequal batches with pages and slots used again, far
keys and bucket edges, the first tokens, long decoding, other sizes, and greedy generation through the entry point.
Weights come from tests/mivorax_configs.py, which makes them so that a lost key, state, sink or bias shows."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import mivorax_configs as mc
import plain_mivorax as pm
import replay_util as ru

pytestmark = pytest.mark.gpu

# a row's error: root mean square of the difference of the logits (mean taken off) over that of the plain logits
LIMIT = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["fp32", "bf16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("mivorax")
    return {n: mc.write_folder(os.path.join(str(root), n), cfg, seed=11 + i, drop_bias_buckets=(n == "mixed_a"))
            for i, (n, cfg) in enumerate(mc.CONFIGS.items())}


@pytest.fixture(scope="module")
def plains(folders):
    return {n: ru.PlainLogits(d, pm) for n, d in folders.items()}


def replayer(folder, name, dtype, max_tokens, max_requests=4):
    from llm_steadyinfer_b200.engine.replay import Replayer
    return Replayer(folder, dtype, max_tokens, page_size=mc.PAGE_SIZE[name], max_requests=max_requests)


def row_error(row, ref):
    d = row.to(torch.float64) - ref
    d = d - d.mean()
    return (d.pow(2).mean().sqrt() / ref.sub(ref.mean()).pow(2).mean().sqrt()).item()


def check(rp, steps, reqs, plain, dtype, what):
    worst, n = 0.0, 0
    for rid, p, row in ru.replay_in_process(rp, steps):
        e = row_error(row, plain.of(reqs[rid])[p])
        assert e == e and e <= LIMIT[dtype], f"{what}: request {rid!r} position {p}: error {e:.3e} (allowed {LIMIT[dtype]:.0e})"
        worst, n = max(worst, e), n + 1
    assert n > 0
    mgr = rp.runner.manager
    mgr.check_invariant()
    assert not mgr.requests
    assert all(mgr.free_pages(g) == mgr.groups[g].pool.num_pages for g in range(len(mgr.groups)))
    return worst


def requests_of(name, lengths, seed=0):
    vocab = mc.CONFIGS[name]["vocab"]
    return {f"q{i}": ru.random_tokens(vocab, n, 1000 * seed + i) for i, n in enumerate(lengths)}


# ---- each mechanism alone, and the layers of a whole model one by one ------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["attention", "latent", "ssm", "pair_mlp"])
def test_each_mechanism_alone(folders, plains, name, dtype):
    """One-layer models: the residual stream after the layer and the logits, whole and token by token."""
    reqs = requests_of(name, [1, 2, 37, 90])
    for mode, steps in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail(reqs, tail=20))):
        rp = replayer(folders[name], name, dtype, 128)
        check(rp, steps, reqs, plains[name], dtype, f"{name}/{mode}")


@pytest.mark.parametrize("name", ["mixed_a", "mixed_b"])
def test_layers_one_by_one_in_32_bit(folders, name):
    """The residual stream after every layer run against the plain one (shared-weight runs counted each time)."""
    toks = ru.random_tokens(mc.CONFIGS[name]["vocab"], 45, 5)
    cfg, w = pm.read_model_folder(folders[name])
    _, want = pm.forward(cfg, w, toks, return_layers=True)
    rp = replayer(folders[name], name, torch.float32, 64)
    got = {}
    rp.runner.model.hook_layers(lambda run, resid: got.__setitem__(run, resid.double().cpu()))
    rp.run_step([{"id": "a", "tokens": toks, "want": [len(toks) - 1]}], end=["a"])
    assert sorted(got) == list(range(len(cfg["layers"])))
    for run in range(len(cfg["layers"])):
        scale = want[run].abs().max().item()
        diff = (got[run] - want[run]).abs().max().item()
        assert diff <= 5e-5 * scale, f"{name}: layer run {run} ({cfg['layers'][run]['type']}) differs by {diff:.2e} of {scale:.1f}"


# ---- schedules ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["mixed_a", "mixed_b", "odd"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_schedules(folders, plains, name, dtype, mode):
    reqs = requests_of(name, [1, 3, 19, 64, 65, 130, 201], seed=1)
    longest = ru.round64(max(len(t) for t in reqs.values()))
    if mode == "whole":
        steps, max_tokens = ru.trace_whole(reqs), longest
    elif mode == "tail":
        steps, max_tokens = ru.trace_tail(reqs, tail=40), longest
    elif mode == "portions":
        steps, max_tokens = ru.trace_portions(reqs, sizes=(2, 17, 3, 2, 31, 5, 64, 2, 9, 1, 40)), longest
    else:
        max_tokens = longest + 128                       # two or three live at a time: pages and slots come again
        steps = ru.trace_mixed(reqs, max_tokens, seed=3, max_live=3)
    rp = replayer(folders[name], name, dtype, max_tokens, max_requests=3)
    worst = check(rp, steps, reqs, plains[name], dtype, f"{name}/{mode}")
    print(f"{name} {mode} {dtype}: worst row error {worst:.2e}")


def test_batch_equals_alone_and_slots_come_again(folders, plains):
    """Unequal requests in one batch against each alone, with two state slots for five requests: every slot and page
    is used again, and what the request before left there (recurrent state, last token, keys) must not show."""
    name, dtype = "mixed_a", torch.float32
    reqs = requests_of(name, [70, 9, 33, 2, 51], seed=2)
    steps = ru.trace_mixed(reqs, 192, seed=9, max_live=2, prompt_frac=0.5)
    rp = replayer(folders[name], name, dtype, 192, max_requests=2)
    check(rp, steps, reqs, plains[name], dtype, "two slots")
    # the same requests once more through the same engine, in another order: slots hold stale state of others now
    again = dict(reversed(list(reqs.items())))
    check(rp, ru.trace_mixed(again, 192, seed=10, max_live=2, prompt_frac=0.3), again, plains[name], dtype, "two slots again")


def test_long_decoding(folders, plains):
    """A short prompt, then 300 tokens one by one, across many page borders and past every bucket of the bias
    tables; the recurrent state is carried 300 times."""
    name = "mixed_a"
    reqs = requests_of(name, [310], seed=3)
    for dtype in DTYPES:
        rp = replayer(folders[name], name, dtype, 320)
        check(rp, ru.trace_tail(reqs, tail=300), reqs, plains[name], dtype, "long decoding")


def test_first_tokens(folders, plains):
    """Positions 0, 1, 2 alone and as the start of portions: the pair embedding's extra row, the convolution's zeros
    before the sequence, a softmax over one key and a sink."""
    name = "mixed_b"
    reqs = requests_of(name, [1, 2, 3, 5], seed=4)
    for dtype in DTYPES:
        for sizes in ((1,), (2, 1), (1, 2)):
            rp = replayer(folders[name], name, dtype, 64)
            check(rp, ru.trace_portions(reqs, sizes=sizes), reqs, plains[name], dtype, f"first tokens {sizes}")


# ---- kernels with inputs that make one key count -----------------------------------------------------------

def _paged(keys, page_size, perm_seed):
    """keys [n, KV, d] into a shuffled page pool; returns (cache [pages, KV, page_size, d], table [1, blocks])."""
    n, KV, d = keys.shape
    blocks = -(-n // page_size)
    g = torch.Generator().manual_seed(perm_seed)
    pages = torch.randperm(blocks + 3, generator=g)[:blocks]
    cache = torch.zeros(blocks + 3, KV, page_size, d, dtype=keys.dtype)
    for j in range(n):
        cache[pages[j // page_size], :, j % page_size] = keys[j]
    return cache, pages.to(torch.int32).view(1, -1)


def _built_attention(case, dtype):
    """Queries, keys and values in which one key far back (and keys at page borders, and at both sides of every bucket
    edge of the bias) carries nearly all the weight of some query; plain result in float64."""
    torch.manual_seed(1)
    n, H, KV, dk, ps = 700, 4, 2, 32, 16
    dv = 48 if case == "bias" else 24
    if case == "sink_latent":
        KV = 1
    k = torch.randn(n, KV, dk) * 0.3
    v = torch.randn(n, KV, dv)
    q = torch.randn(n, H, dk) * 0.3
    rows, dmax = 12, 300.0
    rel = torch.randn(rows, H) * 3.0
    edges = sorted({0, 1, rows // 2 - 1, rows // 2} | {d for d in range(1, 340) if pm.distance_bucket(d, rows, dmax) != pm.distance_bucket(d - 1, rows, dmax)}
                   | {299, 300, 301, 15, 16, 17, 63, 64, 65, 640})
    for e, dist in enumerate(edges):                      # query i = 650 + e looks hard at the key `dist` back
        i = 650 + e
        if i >= n or i - dist < 0:
            continue
        for h in range(H):
            g = h // (H // KV)
            q[i, h] = k[i - dist, g] / k[i - dist, g].norm() * 9.0
        k[i - dist] = k[i - dist] / k[i - dist].norm(dim=-1, keepdim=True) * 9.0
    q, k, v = (t.to(dtype).float() for t in (q, k, v))
    sink = torch.tensor([-2.0, 0.5, 3.0, 40.0])
    scale = 0.7
    ref = torch.zeros(n, H, dv, dtype=torch.float64)
    by_distance = torch.tensor([pm.distance_bucket(d, rows, dmax) for d in range(n)])
    idx = by_distance[(torch.arange(n)[:, None] - torch.arange(n)[None, :]).clamp(min=0)]
    for h in range(H):
        g = h // (H // KV)
        vv = v[:, g] if case == "bias" else k[:, g, :dv]
        bias = rel[:, h].double()[idx] if case == "bias" else None
        ref[:, h] = pm.softmax_attention(q[:, h].double(), k[:, g].double(), vv.double(), scale, bias=bias,
                                         sink=None if case == "bias" else sink[h].double())
    return dict(n=n, H=H, KV=KV, dk=dk, dv=dv, ps=ps, q=q, k=k, v=v, rel=rel, dmax=dmax, sink=sink, scale=scale, ref=ref)


@pytest.mark.parametrize("kernel,dtype", [("general", torch.float32), ("general", torch.bfloat16), ("flex", torch.bfloat16)],
                         ids=["general-fp32", "general-bf16", "flex-bf16"])
@pytest.mark.parametrize("case", ["bias", "sink_latent"])
def test_attention_kernels_far_keys_and_edges(case, kernel, dtype):
    """The general attention kernels (plain and tensor-core) on built inputs; the tensor-core one as portions, and its
    last rows once more as single rows with their keys cut into shares that a second kernel merges."""
    from llm_steadyinfer_b200.csrc import ops
    from llm_steadyinfer_b200.parts.attention import spread_by_distance
    dev = "cuda:0"
    b = _built_attention(case, dtype)
    n, H, KV, dk, dv, ps = b["n"], b["H"], b["KV"], b["dk"], b["dv"], b["ps"]
    kc, table = _paged(b["k"].to(dtype), ps, 3)
    vc = _paged(b["v"].to(dtype), ps, 3)[0].to(dev) if case == "bias" else None
    bias = spread_by_distance(b["rel"], b["dmax"]).to(dev) if case == "bias" else None
    sink = b["sink"].to(dev) if case != "bias" else None
    qd = b["q"].to(dtype).view(n, H * dk).to(dev)
    limit = 1e-4 if dtype == torch.float32 else 3e-2
    out = torch.zeros(n, H * dv, dtype=dtype, device=dev)
    if kernel == "general":
        ops.attention_general(qd, kc.to(dev), vc, table.to(dev), torch.zeros(n, dtype=torch.int32, device=dev),
                              torch.arange(n, dtype=torch.int32, device=dev), out, ps, 1, H, KV, dk, dv, b["scale"], 0,
                              dist_bias=bias, sink=sink)
    else:
        per = ops.attn_flex_tokens(H, KV)
        items = torch.tensor([(0, r, min(per, n - r), r) for r in range(0, n, per)], dtype=torch.int32, device=dev)
        ops.attn_flex(qd, kc.to(dev), vc, table.to(dev), items, out, ps, 1, H, KV, dk, dv, b["scale"], 0, dist_bias=bias, sink=sink)
        ones = torch.tensor([(0, r, 1, r) for r in range(600, n)], dtype=torch.int32, device=dev)
        again = torch.zeros_like(out)
        scratch = torch.zeros(ops.attn_flex_scratch_floats(ones.shape[0], H, KV, dv, 5), dtype=torch.float32, device=dev)
        ops.attn_flex(qd, kc.to(dev), vc, table.to(dev), ones, again, ps, 1, H, KV, dk, dv, b["scale"], 0, dist_bias=bias, sink=sink,
                      nsplit=5, scratch=scratch, max_rows=H // KV)
        diff = (again[600:].double().cpu().view(-1, H, dv) - b["ref"][600:]).abs().max().item()
        assert diff <= limit, f"{case}: rows in shares differ by {diff:.2e}"
    diff = (out.double().cpu().view(n, H, dv) - b["ref"]).abs().max().item()
    assert diff <= limit, f"{case}: differs by {diff:.2e}"
    if case != "bias":        # a sink far above every score leaves almost nothing (rows from 650 on hold the built queries)
        assert out.view(n, H, dv)[:600, 3].abs().max().item() < 1e-6


@pytest.mark.parametrize("H,KV,dk,dv,own_v", [(8, 2, 64, 32, True), (4, 1, 48, 80, True), (16, 1, 160, 128, False),
                                              (128, 1, 72, 64, False), (6, 3, 192, 160, True), (2, 1, 576, 512, False), (16, 1, 320, 288, False)])
def test_tensor_core_attention_sizes(H, KV, dk, dv, own_v):
    """The tensor-core kernel against the plain one at head layouts that take its different routes: value slices, key
    tiles of 32, more heads than a tile has rows, sizes that are no multiple of 16."""
    from llm_steadyinfer_b200.csrc import ops
    dev = "cuda:0"
    torch.manual_seed(H + dk)
    n, ps = 150, 16
    k = (torch.randn(n, KV, dk) * 0.5).bfloat16()
    v = torch.randn(n, KV, dv).bfloat16() if own_v else None
    q = (torch.randn(n, H * dk) * 0.5).bfloat16().to(dev)
    kc, table = _paged(k, ps, 5)
    vc = _paged(v, ps, 5)[0].to(dev) if own_v else None
    sink = torch.randn(H, device=dev)
    bias = torch.randn(40, H, device=dev)
    want = torch.zeros(n, H * dv, dtype=torch.bfloat16, device=dev)
    seqs, pos = torch.zeros(n, dtype=torch.int32, device=dev), torch.arange(n, dtype=torch.int32, device=dev)
    ops.attention_general(q, kc.to(dev), vc, table.to(dev), seqs, pos, want, ps, 1, H, KV, dk, dv, dk ** -0.5, 0, dist_bias=bias, sink=sink)
    per = ops.attn_flex_tokens(H, KV)
    items = torch.tensor([(0, r, min(per, n - r), r) for r in range(0, n, per)], dtype=torch.int32, device=dev)
    got = torch.zeros_like(want)
    ops.attn_flex(q, kc.to(dev), vc, table.to(dev), items, got, ps, 1, H, KV, dk, dv, dk ** -0.5, 0, dist_bias=bias, sink=sink)
    assert (got.float() - want.float()).abs().max().item() <= 2e-2
    ones = torch.tensor([(0, r, 1, r) for r in range(n)], dtype=torch.int32, device=dev)
    scratch = torch.zeros(ops.attn_flex_scratch_floats(n, H, KV, dv, 3), dtype=torch.float32, device=dev)
    got.zero_()
    # single rows with key shares; the caller says how many rows an item has at most (few rows over keys that are
    # their own values: the warps take a value slice each)
    ops.attn_flex(q, kc.to(dev), vc, table.to(dev), ones, got, ps, 1, H, KV, dk, dv, dk ** -0.5, 0, dist_bias=bias, sink=sink, nsplit=3,
                  scratch=scratch, max_rows=min(H // KV, 64))
    assert (got.float() - want.float()).abs().max().item() <= 2e-2
    got.zero_()
    ops.attn_flex(q, kc.to(dev), vc, table.to(dev), ones, got, ps, 1, H, KV, dk, dv, dk ** -0.5, 0, dist_bias=bias, sink=sink,
                  max_rows=min(H // KV, 64))
    assert (got.float() - want.float()).abs().max().item() <= 2e-2


def test_bias_table_is_spread_as_the_plain_bucket_says():
    from llm_steadyinfer_b200.parts.attention import spread_by_distance
    for rows, dmax in ((2, 5.0), (6, 9.0), (12, 300.0), (32, 120.0), (16, 17.5), (10, 1000.0)):
        rel = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
        got = spread_by_distance(rel, dmax)
        for n in range(int(dmax) + 50):
            assert torch.equal(got[min(n, got.shape[0] - 1)], rel[pm.distance_bucket(n, rows, dmax)]), (rows, dmax, n)


@pytest.mark.parametrize("heads,P,N,groups,taps", [(4, 24, 16, 2, 4), (3, 64, 128, 1, 2), (2, 8, 5, 2, 1), (6, 48, 48, 3, 5)])
def test_state_space_kernels_in_portions(heads, P, N, groups, taps):
    """Convolution, recurrence and gated norm over one sequence cut into portions (2, 1, 17, ...) beside a second
    sequence, against the plain functions on the whole sequence; the slot starts with another request's leavings."""
    from llm_steadyinfer_b200.csrc import ops
    dev = "cuda:0"
    torch.manual_seed(heads * 100 + N)
    T = 84
    inner, C = heads * P, heads * P + 2 * groups * N
    u = torch.randn(T, C + heads + inner)                     # [z | xBC | dt] rows as the projection lays them out
    conv_w, conv_b = torch.randn(C, taps) * 0.5, torch.randn(C) * 0.1
    dt_bias, a_log, dsk = torch.empty(heads).uniform_(-4, -1), torch.empty(heads).uniform_(-1, 1), torch.randn(heads)
    norm_w = 1 + 0.1 * torch.randn(inner)
    z, xbc_in, dt_raw = u[:, :inner], u[:, inner:inner + C], u[:, inner + C:]
    xbc = pm.silu(pm.causal_conv(xbc_in.double(), conv_w.double(), conv_b.double()))
    y = pm.state_space_scan(xbc[:, :inner].contiguous(), xbc[:, inner:inner + groups * N].contiguous(), xbc[:, inner + groups * N:].contiguous(),
                            pm.softplus(dt_raw.double() + dt_bias.double()), a_log.double(), dsk.double(), heads, groups)
    want = pm.rms_norm((y * pm.silu(z.double())).view(T, 2, inner // 2), None, 1e-5).reshape(T, inner) * norm_w.double()
    assert ops.ssm_padded_state(N, P) == ops.ssm_padded_state_of_library(N, P)
    conv_off = heads * ops.ssm_padded_state(N, P) * P
    state = torch.randn(3, conv_off + (taps - 1) * C, device=dev)          # stale contents
    got = torch.zeros(T, inner, device=dev)
    ud = u.to(dev)
    other = torch.randn(40, u.shape[1], device=dev)
    p = po = 0
    for n in (2, 1, 17, 3, 30, 1, 1, 29):
        no = min(5, 40 - po)
        rows = torch.cat([other[po:po + no], ud[p:p + n]])                    # the other sequence first, in slot 2
        R = rows.shape[0]
        ints = lambda *v: torch.tensor(v, dtype=torch.int32, device=dev)
        positions = torch.cat([torch.arange(po, po + no), torch.arange(p, p + n)]).to(torch.int32).to(dev)
        row_seq = torch.tensor([0] * no + [1] * n, dtype=torch.int32, device=dev)
        q_start, ctx_len, slots = ints(0, no, R), ints(po + no, p + n), ints(2, 1)
        xo = torch.zeros(R, C, device=dev)
        ops.causal_conv(rows[:, inner:inner + C], conv_w.to(dev), conv_b.to(dev), state, conv_off, xo, positions, row_seq, q_start, ctx_len, slots, 2)
        yo = torch.zeros(R, inner, device=dev)
        ops.ssm_scan(xo, rows[:, inner + C:], dt_bias.to(dev), a_log.to(dev), dsk.to(dev), state, yo, q_start, ctx_len, slots, 2, heads, groups, N, P)
        go = torch.zeros(R, inner, device=dev)
        ops.gated_part_norm(yo, rows[:, :inner], norm_w.to(dev), go, 2, 1e-5)
        got[p:p + n] = go[no:]
        p, po = p + n, po + no
    assert p == T
    diff = (got.double().cpu() - want).abs().max().item()
    assert diff <= 2e-4, f"differs by {diff:.2e}"


# ---- the entry point ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["mixed_a", "mixed_b", "odd"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """Greedy tokens through LLM (scheduler, sampler, graphs and steps launched ahead where the model allows) equal the
    plain implementation's in 32-bit; bfloat16 runs and mostly agrees."""
    from llm_steadyinfer_b200 import LLM, SamplingParams
    cfg, w = pm.read_model_folder(folders[name])
    prompts = [ru.random_tokens(cfg["vocab"], n, 50 + n) for n in (5, 23, 1, 40)]
    want = [pm.generate(cfg, w, p, 12) for p in prompts]
    for dtype in ("float32", "bfloat16"):
        for graphs in (True, False):
            llm = LLM(folders[name], dtype=dtype, max_batch=3, max_seq_len=64, max_gen_len=12, block_size=mc.PAGE_SIZE[name],
                      max_num_batched_tokens=32, use_cuda_graph=graphs, async_decode=graphs)
            got = [g.token_ids for g in llm.generate(prompts, SamplingParams(ignore_eos=True))]
            if dtype == "float32":
                assert got == want, f"{name} graphs={graphs}: {got} != {want}"
            else:
                same = sum(a == b for g, x in zip(got, want) for a, b in zip(g, x))
                assert same >= 24, f"{name} bf16: only {same} of 48 tokens agree"
            if graphs:
                assert llm.runner.graphs_available() and llm.stats["graph_steps"] > 0


def test_preemption_recomputes_state_from_the_start(folders):
    """A pool too small for all requests: some are cut back and computed again; with per-request state nothing of a
    cut request can be kept, and the tokens still equal the plain implementation's."""
    from llm_steadyinfer_b200 import LLM, SamplingParams
    name = "mixed_a"
    cfg, w = pm.read_model_folder(folders[name])
    prompts = [ru.random_tokens(cfg["vocab"], n, 90 + n) for n in (30, 28, 26)]
    want = [pm.generate(cfg, w, p, 20) for p in prompts]
    llm = LLM(folders[name], dtype="float32", max_batch=3, max_seq_len=64, max_gen_len=20, block_size=8, num_blocks=14,
              max_num_batched_tokens=64)
    res = llm.generate(prompts, SamplingParams(ignore_eos=True))
    assert [r.token_ids for r in res] == want
    assert sum(r.num_preemptions for r in res) > 0


def test_trace_program(folders, plains, tmp_path):
    """bin/trace_run as a program on a mixed trace."""
    name = "mixed_a"
    reqs = requests_of(name, [40, 7, 90], seed=6)
    steps = ru.trace_mixed(reqs, 256, seed=1, max_live=3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "256", "--page-size", str(mc.PAGE_SIZE[name])],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    pos, vocab = {}, mc.CONFIGS[name]["vocab"]
    for rec in steps:
        wanted = sum(len(e["want"]) for e in rec["entries"])
        rows = None
        if wanted:
            rows = torch.from_file(str(out / f"{rec['step']}.f32"), size=wanted * vocab, dtype=torch.float32).view(wanted, vocab)
        r = 0
        for e in rec["entries"]:
            base = pos.get(e["id"], 0)
            for wpos in e["want"]:
                assert row_error(rows[r], plains[name].of(reqs[e["id"]])[base + wpos]) <= LIMIT[torch.float32]
                r += 1
            pos[e["id"]] = base + len(e["tokens"])


@pytest.mark.parametrize("M,H,N,K,a_head,o_head", [(1, 3, 56, 24, 40, 72), (8, 16, 512, 128, 192, 576), (16, 5, 40, 56, 56, 40), (7, 4, 9, 640, 640, 16)])
def test_per_head_product(M, H, N, K, a_head, o_head):
    """One launch for all heads' small matrices against torch, heads lying inside wider rows."""
    from llm_steadyinfer_b200.csrc import ops
    torch.manual_seed(M + H)
    a = torch.randn(M, (H - 1) * a_head + K + 8, device="cuda:0").bfloat16()
    w = (torch.randn(H, N, K, device="cuda:0") / K ** 0.5).bfloat16()
    out = torch.full((M, (H - 1) * o_head + N + 4), 7.0, device="cuda:0").bfloat16()
    assert ops.gemm_heads_ok(a, w, out, H, a_head, o_head)
    ops.gemm_heads(a, w, out, a_head, o_head)
    for h in range(H):
        want = a[:, h * a_head:h * a_head + K].float() @ w[h].float().T
        assert (out[:, h * o_head:h * o_head + N].float() - want).abs().max().item() <= 2e-2
    if o_head > N:
        assert (out[:, N:o_head] == 7.0).all()            # nothing written between the heads


def test_command_line_serves_the_design(folders, tmp_path):
    """The serving program on a Mivorax folder: requests of random lengths arriving over time, sampling, a pool that
    is used again; and once more on random weights drawn from a configuration file."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "m.json"
    common = ["--num-requests", "12", "--max-batch", "4", "--max-gen", "10", "--prompt-len-dist", "lognormal:30,0.7,2,90",
              "--output-len-dist", "lognormal:6,0.5,1,10", "--request-rate", "300", "--temperature", "0.8", "--top-p", "0.9",
              "--ignore-eos", "--kv-block-size", "8", "--num-kv-blocks", "60", "--max-num-batched-tokens", "40",
              "--max-model-len", "128", "--output-json", str(out)]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(mc.MIXED_B))
    for source in (["--checkpoint", folders["mixed_a"]], ["--model-config", str(cfg_file)]):
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "offline_batch_benchmark"), *source, *common],
                              capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-3000:]
        m = json.loads(out.read_text())[0]
        assert m["completed"] == 12 and m["rejected"] == 0 and m["output_tokens"] > 12 and m["output_tps"] > 0


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 5632, 2048), (16, 40, 72), (128, 384, 256), (300, 1000, 136), (2048, 520, 256)])
def test_products_with_the_activation_in_the_epilogue(M, N, K):
    """relu(x W^T)^2 from the few-row product and from the tcgen05 product against the product stored in bfloat16 and
    the activation kernel after it."""
    from llm_steadyinfer_b200.csrc import ops
    from llm_steadyinfer_b200.parts.linear import linear
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda:0").bfloat16()
    w = (torch.randn(N, K, device="cuda:0") / K ** 0.5).bfloat16()
    want = torch.empty(M, N, device="cuda:0", dtype=torch.bfloat16)
    linear(x, w, want)
    ops.activation(want, want, "relu2")
    got = torch.full_like(want, 3.0)
    if M <= 16:
        ops.gemm_skinny_relu2(x, w, got)
    else:
        ops.gemm_tc05_relu2(x, w, got)
    ref = torch.relu(x.float() @ w.float().T) ** 2
    assert (got.float() - ref).abs().max().item() <= 0.05 * max(1.0, ref.abs().max().item())
    assert (got.float() - want.float()).abs().max().item() <= 0.02 * max(1.0, ref.abs().max().item())
