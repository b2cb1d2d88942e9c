"""Gudarax on the device against its plain statement (tests/plain_gudarax.py, float64, whole sequences).

Whole models: the residual after every layer; every way of cutting the work (whole prompts, a tail decoded token by token,
portions down to two tokens and one, mixed batches whose pages and state slots are used again), bit for bit against one
another in 32-bit; long decoding past every window; decoding from captured graphs; greedy generation through the scheduler;
the trace runner.  Mechanisms alone: attention with a bias by distance at every edge of its window (one key made to stand
out just inside and just outside, far back, at page borders, pages in scrambled order, all three kernels), projection
biases and blended values on their way into the pages, the delta rule's convolutions, unit norms, decays and recurrence
across portions (a write far back read much later), the router's sigmoid scores and the experts whose inputs carry the
scores (few rows and many), the token's own input.
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gudarax as plain
import traces
from gudarax_configs import CONFIGS, write_folder
from helpers import folder_weights, max_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def runner_for(folder, dtype, page_size, pages, slots=4, poison=True):
    from wllm_b200.config import EngineConfig
    from wllm_b200.engine import build_model, build_runner
    eng = EngineConfig(dtype=dtype, block_size=page_size, max_num_seqs=slots)
    return build_runner(build_model(folder, eng.dtype, eng.device), eng, num_pages=pages, poison_pages=poison)


def plain_rows(folder, name, reqs):
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    return {(rid, p): row.float() for rid, toks in reqs.items() for p, row in enumerate(plain.forward(CONFIGS[name], w, toks))}


def close_enough(rows, ref, dtype, what=""):
    """32-bit: every logit within 2e-4 of the logits' scale.  bfloat16: every row's root-mean-square difference against the
    rows' scale: the typical row within 1.5 %, 97 of 100 rows within 6 % (where two experts' scores nearly tie, the rounded
    input may choose the other one, in any implementation: single rows far off, about one in a hundred with these weights)."""
    assert set(rows) == set(ref)
    scale = max(1.0, max(float(r.abs().max()) for r in ref.values()))
    if dtype == torch.float32:
        assert max_diff(rows, ref) < 2e-4 * scale, what
        return
    rms = math.sqrt(sum(float(r.double().pow(2).mean()) for r in ref.values()) / len(ref))
    rel = sorted(float((rows[k].double() - ref[k].double()).pow(2).mean().sqrt()) / rms for k in ref)
    assert rel[len(rel) // 2] < 0.015 and rel[int(0.97 * len(rel))] < 0.06, (what, rel[len(rel) // 2], rel[int(0.97 * len(rel))], rel[-1])


def requests_of(name, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in CONFIGS:
        folder = write_folder(str(tmp_path_factory.mktemp("gudarax") / name), name)
        reqs = requests_of(name, (5, 64, 31, 90, 2, 47, 70, 25, 1, 113, 17), seed=3)
        out[name] = (folder, reqs, plain_rows(folder, name, reqs))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_residual_after_every_layer(setups, name, dtype):
    from wllm_b200.engine import StepEntry
    folder, reqs, _ = setups[name]
    toks = reqs["r3"]
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    want = []
    plain.forward(CONFIGS[name], w, toks, want)
    runner = runner_for(folder, dtype, 16, 8)
    model, got = runner.model, []

    class Watched:
        def __init__(self, block):
            self.block = block

        def __getattr__(self, key):
            return getattr(self.block, key)

        def __call__(self, residual, ctx, cache):
            self.block(residual, ctx, cache)
            p = residual.pending
            if hasattr(p, "materialize"):
                add = p.materialize(ctx, "watched_branch")
            else:
                add = p.tensor.sum(0) if hasattr(p, "tensor") else p
            got.append((residual.stream + add.float()).double().cpu())
    blocks = model.blocks
    model.blocks = [Watched(b) for b in blocks]
    rc = runner.cache.open("x")
    runner.step([StepEntry(rc, toks, [0])])
    model.blocks = blocks
    assert len(got) == len(CONFIGS[name]["layers"])
    for run, (a, b) in enumerate(zip(got, want)):
        tol = (2e-5 if dtype == torch.float32 else 0.03) * float(b.abs().max())
        worst = (a - b).abs().amax(-1).sort().values
        # (bfloat16 is judged by rows: where two experts' scores nearly tie, the rounded input may choose the other one)
        at = len(worst) - 1 if dtype == torch.float32 else int(0.9 * len(worst))
        assert worst[at] < tol, (run, float(worst[at]), float(worst[-1]), tol)


CUTS = (("whole", traces.whole), ("tail", lambda r: traces.tail_singly(r, 16)), ("portions", traces.portions),
        ("mixed", lambda r: traces.mixed(r, seed=5)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_matches_the_plain_statement(setups, name, dtype):
    folder, reqs, ref = setups[name]
    first = None
    for cut, make in CUTS:
        steps = make(reqs)
        pages = -(-traces.peak_tokens(steps) // 16)
        runner = runner_for(folder, dtype, 16, pages)       # four state slots for eleven requests: slots are used again
        rows = traces.run_in_process(runner, steps)
        close_enough(rows, ref, dtype, cut)
        assert all(f == pages for f in runner.cache.free_pages())
        if cut == "mixed":      # pages were used again
            assert all(g.pool.takes > pages for g in runner.cache.groups if g.spec.window is None) and len(reqs) > 4
        if dtype == torch.float32:
            if first is None:
                first = rows
            else:
                bad = sorted(k for k in first if not torch.equal(first[k], rows[k]))
                assert not bad, f"{cut}: first differing (request, position) {bad[0]}"


@pytest.mark.parametrize("page", [32, 64])
def test_other_page_sizes_give_the_same_rows(setups, page):
    folder, reqs, ref = setups["mixed"]
    steps = traces.mixed(reqs, seed=9)
    runner = runner_for(folder, torch.float32, page, -(-traces.peak_tokens(steps, page if page > 64 else 64) // page))
    close_enough(traces.run_in_process(runner, steps), ref, torch.float32, f"pages of {page}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["mixed", "odd", "heads64"])
def test_long_decoding_passes_every_window_and_gives_pages_back(setups, name, dtype):
    from wllm_b200.engine import StepEntry
    folder = setups[name][0]
    reqs = requests_of(name, (230,), seed=8)
    ref = plain_rows(folder, name, reqs)
    steps = traces.tail_singly(reqs, 200)
    runner = runner_for(folder, dtype, 16, 15)          # 15 pages hold 240 tokens
    rc = runner.cache.open("r0")
    rows, pos, held = {}, 0, []
    for s in steps:
        e = s["entries"][0]
        logits = runner.step([StepEntry(rc, e["tokens"], e["want"])]).float().cpu()
        rows.update({("r0", pos + w): row for w, row in zip(e["want"], logits)})
        pos += len(e["tokens"])
        held.append([sum(1 for p in t if p >= 0) for t in rc.tables])
    close_enough(rows, ref, dtype)
    for g, spec in enumerate(runner.model.group_specs):
        if spec.window is not None:      # a group with a window holds the pages that its rule still needs, no more
            most = -(-spec.window // 16) + 1
            assert max(h[g] for h in held[60:]) <= most < 15, (spec, held[-1])
    runner.cache.close(rc)
    assert all(f == 15 for f in runner.cache.free_pages())


def test_decoding_from_captured_graphs_gives_the_eager_rows(setups):
    folder, reqs, ref = setups["mixed"]
    some = {k: reqs[k] for k in ("r1", "r2", "r5")}
    steps = traces.tail_singly(some, 30)
    rows = {}
    for graphs in (False, True):
        runner = runner_for(folder, torch.float32, 16, -(-traces.peak_tokens(steps) // 16), poison=False)
        assert runner.model.graph_safe
        if graphs:
            runner.enable_graphs()
        rows[graphs] = traces.run_in_process(runner, steps)
        assert (runner.graph_launches > 0) == graphs
        close_enough(rows[graphs], {k: v for k, v in ref.items() if k[0] in some}, torch.float32)
    bad = sorted(k for k in rows[False] if not torch.equal(rows[False][k], rows[True][k]))
    assert not bad, f"first differing (request, position) {bad[0]}"


def test_greedy_generation_through_the_scheduler(setups):
    from wllm_b200 import LLM, SamplingParams
    folder, reqs, _ = setups["mixed"]
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    prompts = [reqs["r0"], reqs["r2"], reqs["r3"][:40], reqs["r8"]]
    llm = LLM(folder, dtype="float32", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True))
    for prompt, o in zip(prompts, outs):
        toks = list(prompt)
        for _ in range(30):
            toks.append(int(plain.forward(CONFIGS["mixed"], w, toks)[-1].argmax()))
        assert o.token_ids == toks[len(prompt):]
    assert all(f == 12 for f in llm.runner.cache.free_pages())
    bf = LLM(folder, dtype="bfloat16", block_size=16, num_blocks=12, chunked_prefill_tokens=24, max_num_seqs=3, cuda_graphs=True)
    assert [len(o.token_ids) for o in bf.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))] == [10] * 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_replays_a_mixed_trace(setups, tmp_path, dtype):
    folder, reqs, ref = setups["heads64"]
    steps = traces.mixed(reqs, seed=11)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(traces.peak_tokens(steps))], input="".join(json.dumps(s) + "\n" for s in steps),
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    rows, pos = {}, {}
    V = CONFIGS["heads64"]["vocab"]
    for s in steps:
        keys = []
        for e in s["entries"]:
            p = pos.get(e["id"], 0)
            keys += [(e["id"], p + w) for w in e["want"]]
            pos[e["id"]] = p + len(e["tokens"])
        data = np.fromfile(str(out / f"{s['step']}.f32"), dtype="<f4").reshape(len(keys), V)
        rows.update({k: torch.from_numpy(r.copy()) for k, r in zip(keys, data)})
    close_enough(rows, ref, torch.float32 if dtype == "float32" else torch.bfloat16)


# ------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------
class Scratch:
    """Stands in for the step context where a part is run alone: buffers by name, the step's index arrays as given."""

    def __init__(self, **arrays):
        self.bufs, self.memo = {}, {}
        self.__dict__.update(arrays)

    def buffer(self, name, shape, dtype):
        key = (name, tuple(shape), dtype)
        if key not in self.bufs:
            self.bufs[key] = torch.empty(tuple(shape), dtype=dtype, device=DEV)
        return self.bufs[key]


def paged(rows_k, rows_v, page_size, order_seed, spare=3):
    """Keys [L, G, d] and values [L, G, dv] of one sequence on pages in scrambled order, NaN wherever no token lies."""
    L, G, d = rows_k.shape
    pages = -(-L // page_size)
    perm = torch.randperm(pages + spare, generator=torch.Generator().manual_seed(order_seed))[:pages]
    kp = torch.full((pages + spare, G, page_size, d), float("nan"), dtype=rows_k.dtype)
    vp = torch.full((pages + spare, G, page_size, rows_v.shape[-1]), float("nan"), dtype=rows_k.dtype)
    for j in range(L):
        kp[perm[j // page_size], :, j % page_size] = rows_k[j]
        vp[perm[j // page_size], :, j % page_size] = rows_v[j]
    return kp.to(DEV), vp.to(DEV), perm.to(torch.int32)[None].contiguous().to(DEV)


def plain_window_rows(q, k, v, positions, scale, window, slopes):
    """q [n, H, d] at `positions` over keys k [L, G, d] and values v [L, G, dv]: softmax of scale q.k - slope_h (p - j) over
    the keys p - window < j <= p."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for r, p in enumerate(positions):
        j = torch.arange(k.shape[0])
        seen = (j <= p) & ((j > p - window) if window else True)
        heads = []
        for a in range(H):
            s = (k[:, a // (H // G)].double() @ q[r, a].double()) * scale - slopes[a] * (p - j).double()
            heads.append(torch.softmax(s.masked_fill(~seen, float("-inf")), 0) @ v[:, a // (H // G)].double())
        out.append(torch.cat(heads))
    return torch.stack(out)


def three_kernels(qd, kp, vp, table, positions, L, H, G, d, dv, ps, window, scale, dtype, slopes):
    """The walk, the split and the tiled kernel on the same rows (one portion of one request), and the last row alone."""
    from wllm_b200.kernels import ops
    n = len(positions)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    req = torch.zeros(n, dtype=torch.int32, device=DEV)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    more = dict(vd=dv, slopes=slopes)
    outs = []
    for kind in ("walk", "split", "tiled"):
        out = torch.empty(n, H * dv, dtype=dtype, device=DEV)
        if kind == "tiled":
            ops.paged_attention_simt_tiled(qd, out, kp, vp, one(0), one(n), one(L), table, n, H, G, d, ps, window, scale, **more)
        else:
            chunks = ops.simt_chunks(L, window)
            scratch = torch.empty(n * H * chunks * (dv + 2), device=DEV) if kind == "split" else None
            ops.paged_attention_simt(qd, out, kp, vp, req, pos_t, table, H, G, d, ps, window, scale, scratch, chunks, **more)
        outs.append(out.cpu())
    last = torch.empty(1, H * dv, dtype=dtype, device=DEV)
    ops.paged_attention_simt(qd[-1:], last, kp, vp, req[:1], pos_t[-1:], table, H, G, d, ps, window, scale, **more)
    return outs, last.cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [40, 64, 17, 1, 130, 0])
def test_attention_with_a_bias_by_distance_at_every_edge_of_its_window(window, dtype):
    """One key at a time is made to stand out (along the query, long enough to take all the weight where it is seen): the key
    just outside the first row's window and the one just inside, the same for the last row, the rows' own positions, keys at
    page and chunk borders and key 0 far back.  Rows of a prompt's portion and a single decoded row, pages in scrambled
    order, all three kernels, whose results are one, bit for bit.  Window 0: every earlier key, a far key among hundreds.
    The slopes are steep enough for the bias to decide between near and far keys, and differ from head to head."""
    g = torch.Generator().manual_seed(window * 7 + 1)
    H, G, d, dv, ps, L = 4, 2, 16, 24, 16, 300
    scale = 0.4
    slopes = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    k, v = torch.randn(L, G, d, generator=g).to(dtype), torch.randn(L, G, dv, generator=g).to(dtype)
    n0 = 236
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, d, generator=g).to(dtype)
    first = (lambda p: max(0, p - window + 1)) if window else (lambda p: 0)
    edges = sorted({e for e in (0, 1, first(n0) - 1, first(n0), first(n0) + 1, n0 - 1, n0, first(L - 1) - 1, first(L - 1), 63, 64, 255, 256, 239, 240)
                    if 0 <= e < L})
    sl = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(DEV)
    base = plain_window_rows(q, k, v, positions, scale, window, slopes)
    changed = 0
    for edge in edges:
        k2 = k.clone()
        k2[edge] = (q[-1, 0].float() * 6).to(dtype)[None].expand(G, d)       # along the last row's first query: it takes the weight
        want = plain_window_rows(q, k2, v, positions, scale, window, slopes)
        changed += int((want - base).abs().max() > 0.1)
        kp, vp, table = paged(k2, v, ps, edge + 5)
        (walk, split, tiled), last = three_kernels(q.reshape(len(positions), H * d).to(DEV), kp, vp, table, positions, L, H, G, d, dv, ps,
                                                   window, scale, dtype, sl)
        assert torch.equal(walk, split) and torch.equal(walk, tiled) and torch.equal(walk[-1:], last), edge
        tol = 2e-5 if dtype == torch.float32 else 0.02
        assert (walk.double() - want).abs().max() < tol * max(1.0, float(want.abs().max())), (edge, float((walk.double() - want).abs().max()))
    assert changed >= 3 or window == 1         # the keys made to stand out do decide rows where they are seen
    # the bias alone decides: without it the far key wins, with it the near one
    flat = plain_window_rows(q, k, v, positions, scale, window, [0.0] * H)
    assert window == 1 or (flat - base).abs().max() > 1e-3


@pytest.mark.parametrize("hd,n0", [(32, 236), (64, 236), (64, 100), (128, 150)])
@pytest.mark.parametrize("window", [40, 17, 130, 0])
def test_tensor_core_attention_with_a_bias_by_distance(window, hd, n0):
    """The bfloat16 kernels on mma.sync with slopes: a prompt's portion over several tiles of rows and decoded rows of three
    requests whose keys are cut into splits, one key standing out at every edge of the window, pages of 16 and 64 in
    scrambled order; grouped heads, so that a tile's rows carry different slopes."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(window * 7 + hd)
    H, G, L, dtype = 4, 2, 300, torch.bfloat16
    scale = 0.4 * (16 / hd) ** 0.5
    slopes = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    sl = torch.tensor(slopes, dtype=torch.float32, device=DEV)
    k, v = torch.randn(L, G, hd, generator=g).to(dtype), torch.randn(L, G, hd, generator=g).to(dtype)
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, hd, generator=g).to(dtype)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    first = (lambda p: max(0, p - window + 1)) if window else (lambda p: 0)
    edges = sorted({e for e in (0, first(n0) - 1, first(n0), first(L - 1) - 1, first(L - 1), L - 1, 63, 64, 127, 128) if 0 <= e < L})
    for ps in (16, 64):
        for edge in edges:
            k2 = k.clone()
            k2[edge] = (q[-1, 0] * 6).to(dtype)[None].expand(G, hd)
            kp, vp, table = paged(k2, v, ps, 5 + ps)
            want = plain_window_rows(q, k2, v, positions, scale, window, slopes)
            qd = q.reshape(len(positions), H * hd).to(DEV)
            out = torch.empty(len(positions), H * hd, dtype=dtype, device=DEV)
            ops.attention_mma_prefill(qd, out, kp, vp, one(0), one(len(positions)), one(L), table, len(positions), H, G, hd, ps, window,
                                      scale, skip_single=False, slopes=sl)
            err = (out.cpu().double() - want).abs().max()
            assert err < 0.03, ("prefill", ps, edge, float(err))
            R = 3
            tables = table.expand(R, -1).contiguous()
            starts = torch.arange(R, dtype=torch.int32, device=DEV)
            lens = torch.ones(R, dtype=torch.int32, device=DEV)
            ctxs = torch.tensor([L - 2, L - 1, L], dtype=torch.int32, device=DEV)
            for split_keys, max_splits in ((512, 1), (128, 3), (64, 5)):
                scratch = torch.empty(ops.attention_mma_scratch_floats(R, H, hd, max_splits), device=DEV)
                od = torch.empty(R, H * hd, dtype=dtype, device=DEV)
                ops.attention_mma_decode(qd[-3:].contiguous(), od, kp, vp, starts, lens, ctxs, tables, H, G, hd, ps, window, scale,
                                         split_keys, max_splits, scratch, slopes=sl)
                err = (od.cpu().double() - want[-3:]).abs().max()
                assert err < 0.03, ("decode", ps, edge, split_keys, float(err))
    assert ops.tc_gemm_status(DEV) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24), (5, 1, 10, 6), (2, 2, 64, 64)])
def test_biases_row_norms_and_blended_values_on_their_way_into_the_pages(sizes, dtype):
    """q | k | v from a product (as one tensor, and as 32-bit partial sums), a bias row added, q and k normed as whole rows,
    the values blended with an earlier layer's: what lands in q_out and in the pages, against the formulas."""
    from wllm_b200.kernels import ops
    nq, nkv, hd_file, vd_file = sizes
    hd, vd = -(-hd_file // 8) * 8, -(-vd_file // 8) * 8
    g = torch.Generator().manual_seed(nq * 100 + hd_file)
    n, ps, eps = 37, 16, 1e-5

    def padded(x, heads, size, to):          # [n, heads * size] -> [n, heads * to], zeros behind every head
        out = x.new_zeros((x.shape[0], heads, to))
        out[:, :, :size] = x.view(x.shape[0], heads, size)
        return out.view(x.shape[0], heads * to)
    qf, kf, vf = (torch.randn(n, nq * hd_file, generator=g), torch.randn(n, nkv * hd_file, generator=g), torch.randn(n, nkv * vd_file, generator=g))
    bq, bk, bv = (torch.randn(1, nq * hd_file, generator=g), torch.randn(1, nkv * hd_file, generator=g), torch.randn(1, nkv * vd_file, generator=g))
    gq, gk = 1 + 0.3 * torch.randn(1, nq * hd_file, generator=g), 1 + 0.3 * torch.randn(1, nkv * hd_file, generator=g)
    fused = torch.cat([padded(qf, nq, hd_file, hd), padded(kf, nkv, hd_file, hd), padded(vf, nkv, vd_file, vd)], 1)
    bias = torch.cat([padded(bq, nq, hd_file, hd), padded(bk, nkv, hd_file, hd), padded(bv, nkv, vd_file, vd)], 1)[0].contiguous()
    q_gain = padded(gq, nq, hd_file, hd)[0].to(dtype).contiguous().to(DEV)
    k_gain = padded(gk, nkv, hd_file, hd)[0].to(dtype).contiguous().to(DEV)
    lam = torch.tensor([0.37])
    first = torch.randn(n, nkv * vd, generator=g)
    positions = torch.arange(5, 5 + n, dtype=torch.int32, device=DEV)
    slots = torch.randperm(4 * ps, generator=g)[:n].to(torch.int32).to(DEV)
    none = torch.empty(0, dtype=torch.float32, device=DEV)
    for parts in (0, 3):
        if parts:
            cut = torch.randn(parts, n, fused.shape[1], generator=g)
            cut[0] += fused - cut.sum(0)
            x, src = cut.to(DEV), cut.double().sum(0)
        else:
            x = fused.to(dtype).to(DEV)
            src = x.double().cpu()
        W = src + bias.double()
        qw, kw = nq * hd, nkv * hd
        def row_norm(y, count, gain):           # the mean counts the heads' own elements, not the zeros behind them
            return y / torch.sqrt((y * y).sum(-1, keepdim=True) / count + eps) * gain.cpu().double()
        want_q, want_k = row_norm(W[:, :qw], nq * hd_file, q_gain), row_norm(W[:, qw:qw + kw], nkv * hd_file, k_gain)
        for mix in (None, "first", "later"):
            kp = torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV)
            vp = torch.zeros(4, nkv, ps, vd, dtype=dtype, device=DEV)
            q_out = torch.empty(n, qw, dtype=dtype, device=DEV)
            v_first = first.clone().to(DEV)
            ops.rope_row_norm_kv_write(x, q_out, positions, slots, none, kp, vp, nq, nkv, hd, 0, ps, q_gain, k_gain, eps, nq * hd_file,
                                       nkv * hd_file, in_splits=parts, vd=vd, bias=bias.to(DEV),
                                       **({} if mix is None else dict(v_first=v_first, blend=lam.to(DEV), mix=mix)))
            tol = 1e-5 if dtype == torch.float32 else 0.02
            assert (q_out.double().cpu() - want_q).abs().max() < tol * float(want_q.abs().max())
            want_v = W[:, qw + kw:]
            if mix == "first":
                assert (v_first.double().cpu() - want_v).abs().max() < 1e-5 * float(want_v.abs().max())     # left unrounded for the later layers
            if mix == "later":
                want_v = (1 - 0.37) * want_v + 0.37 * first.double()
                assert torch.equal(v_first.cpu(), first)
            sl = slots.long().cpu()
            got_k = kp.cpu()[sl // ps, :, sl % ps].reshape(n, kw).double()
            got_v = vp.cpu()[sl // ps, :, sl % ps].reshape(n, nkv * vd).double()
            assert (got_k - want_k).abs().max() < tol * float(want_k.abs().max())
            assert (got_v - want_v).abs().max() < tol * float(want_v.abs().max())


def plain_delta_parts(fused, off, H, G, D, V, taps_q, taps_k, taps_v, a_log, dt_bias, unit_eps=1e-6):
    """q, k, v, beta, decay of a whole sequence from its fused projection rows, by the plain statement's functions."""
    n = fused.shape[0]
    GD, HV = G * D, H * V
    q = plain.silu(plain.short_conv(fused[:, off["q"]:off["q"] + GD], taps_q)).view(n, G, D)
    k = plain.silu(plain.short_conv(fused[:, off["k"]:off["k"] + GD], taps_k)).view(n, G, D)
    v = plain.silu(plain.short_conv(fused[:, off["v"]:off["v"] + HV], taps_v)).view(n, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(fused[:, off["b"]:off["b"] + H])
    decay = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(fused[:, off["a"]:off["a"] + H] + dt_bias))
    return q, k, v, beta, decay


def plain_delta_scan(q, k, v, beta, decay):
    n, H, V = v.shape
    G, D = q.shape[1], q.shape[2]
    out = torch.zeros(n, H, V, dtype=q.dtype)
    for a in range(H):
        S = torch.zeros(D, V, dtype=q.dtype)
        for t in range(n):
            S = S * decay[t, a]
            u = beta[t, a] * (v[t, a] - S.T @ k[t, a // (H // G)])
            S = S + torch.outer(k[t, a // (H // G)], u)
            out[t, a] = S.T @ q[t, a // (H // G)]
    return out


@pytest.mark.parametrize("sizes", [(4, 2, 16, 24, 4), (3, 3, 10, 6, 2), (2, 1, 64, 64, 4), (2, 2, 128, 40, 1), (1, 1, 200, 130, 3)])
def test_the_delta_rule_across_portions_and_slots(sizes):
    """Convolutions whose inputs come from the portion before (portions down to one token, shorter than the taps), unit
    norms, step sizes and decays, and the recurrence from and to a state slot: two requests in one batch, cut in different
    ways, against the plain functions on the whole sequences; the outputs do not depend on the cut, bit for bit.  One early
    token writes a large value that a query far behind it still reads (decays near one in one head)."""
    from wllm_b200.kernels import ops
    H, G, D, V, T = sizes
    g = torch.Generator().manual_seed(H * 31 + D)
    GD, HV = G * D, H * V
    off = {"q": 0, "k": GD, "v": 2 * GD, "g": 2 * GD + HV, "b": 2 * GD + 2 * HV, "a": 2 * GD + 2 * HV + H}
    W = 2 * GD + 2 * HV + 2 * H
    lengths = (150, 47)
    seqs = [torch.randn(n, W, generator=g) for n in lengths]
    taps = [torch.randn(c, T, generator=g) * 0.7 for c in (GD, GD, HV)]
    a_log, dt_bias = torch.rand(H, generator=g) * 2 - 1, torch.randn(H, generator=g) * 0.3
    a_log[0] = -6.0                                  # head 0 forgets next to nothing
    seqs[0][3, off["v"]:off["v"] + V] = 30.0         # a large value early on ...
    seqs[0][140, off["q"]:off["q"] + D] = seqs[0][3, off["k"]:off["k"] + D]     # ... and a query far behind along its key
    want = []
    for s in seqs:
        parts = plain_delta_parts(s.double(), off, H, G, D, V, *[t.double() for t in taps], a_log.double(), dt_bias.double())
        want.append(plain_delta_scan(*parts))
    dev = lambda t: t.contiguous().to(DEV)
    d_taps, d_alog, d_bias = [dev(t) for t in taps], dev(a_log), dev(dt_bias)
    results = []
    for cuts in (((150,), (47,)), ((1, 2, 3, 60, 1, 1, 82), (40, 1, 1, 5)), ((2,) * 75, (47,)), ((149, 1), (1,) * 47)):
        slots = 5
        state = torch.full((slots, H, D, V), float("nan"), device=DEV)
        conv = torch.full((slots, max(T - 1, 1), 2 * GD + HV), float("nan"), device=DEV)
        use = (3, 1)
        for s in use:
            state[s].zero_()
            conv[s].zero_()
        outs = [[], []]
        pos, it = [0, 0], 0
        while pos[0] < lengths[0] or pos[1] < lengths[1]:
            rows, starts, lens, slot_ids, who = [], [], [], [], []
            for r in (0, 1):
                if pos[r] < lengths[r] and it < len(cuts[r]):
                    c = cuts[r][it]
                    starts.append(sum(lens))
                    lens.append(c)
                    slot_ids.append(use[r])
                    rows.append(seqs[r][pos[r]:pos[r] + c])
                    who.append(r)
                    pos[r] += c
            it += 1
            if not rows:
                break
            fused = dev(torch.cat(rows))
            n = fused.shape[0]
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
            token_req = i32([j for j, c in enumerate(lens) for _ in range(c)])
            q, k = torch.empty(n, GD, device=DEV), torch.empty(n, GD, device=DEV)
            v, o = torch.empty(n, HV, device=DEV), torch.empty(n, HV, device=DEV)
            beta, decay = torch.empty(n, H, device=DEV), torch.empty(n, H, device=DEV)
            ops.delta_prepare(fused, 0, off, H, G, D, V, T, *d_taps, d_alog, d_bias, token_req, i32(starts), i32(slot_ids), conv, 1e-6,
                              D ** -0.5, q, k, v, beta, decay)
            ops.delta_conv_update(fused, 0, off, H, G, D, V, T, i32(starts), i32(lens), i32(slot_ids), conv)
            ops.delta_scan(q, k, v, beta, decay, state, o, i32(starts), i32(lens), i32(slot_ids), H, G, D, V)
            for j, r in enumerate(who):
                outs[r].append(o[starts[j]:starts[j] + lens[j]].cpu())
        got = [torch.cat(x).view(-1, H, V) for x in outs]
        for r in (0, 1):
            assert (got[r].double() - want[r]).abs().max() < 3e-5 * max(1.0, float(want[r].abs().max())), (cuts, r)
        assert torch.isnan(state[0]).all() and torch.isnan(state[4]).all()          # other slots are left alone
        results.append(got)
    for other in results[1:]:
        assert torch.equal(results[0][0], other[0]) and torch.equal(results[0][1], other[1])


def expert_part(E, top, H, I, dtype, seed):
    from wllm_b200.parts import FEED_FORWARDS, spec
    g = torch.Generator().manual_seed(seed)
    w = {"r": torch.randn(E, H, generator=g) * 0.5}
    for j in range(E):
        w[f"e{j}.up"], w[f"e{j}.down"] = torch.randn(I, H, generator=g) * 0.2, torch.randn(H, I, generator=g) * 0.2
    w = {k: v.to(dtype) for k, v in w.items()}
    part = FEED_FORWARDS.build(spec("routed_experts", num_experts=E, top=top, router="r", expert_prefix="e", intermediate_size=I,
                                    activation="relu_squared", scores="sigmoid", gated=False, weight_on="input"),
                               hidden_size=H, model_dtype=dtype)
    part.load(lambda name: w[name].to(DEV))
    return part, {("router" if k == "r" else k): v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(6, 2, 64, 40, 9), (3, 1, 50, 14, 70), (4, 4, 64, 32, 33), (8, 2, 128, 96, 700)])
def test_experts_whose_inputs_carry_their_sigmoid_scores(sizes, dtype):
    """The chosen experts (the largest sigmoid scores, not normalised), and sum over them of down(relu(up (s x))^2): few rows
    (products that gather rows on the fly) and many (the tensor-memory product over rows copied into sorted order)."""
    from wllm_b200.kernels import ops
    E, top, H, I, n = sizes
    part, w = expert_part(E, top, H, I, dtype, seed=E * 10 + n)
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, H, generator=g).to(dtype)
    mlp = {"router": {"experts": E, "top": top}}
    idx, val = plain.route(mlp, w, "", x.double())
    ctx = Scratch()
    out = part(x.to(DEV), ctx)
    chosen = ctx.bufs[("moe_chosen", (n, top), torch.int32)].cpu().long()
    weights = ctx.bufs[("moe_weights", (n, top), torch.float32)].cpu()
    # a row whose two best scores nearly tie may go either way; everywhere else the choice is the plain statement's
    z = torch.sigmoid(x.double() @ w["router"].T).sort(-1, descending=True).values
    clear = (z[:, top - 1] - z[:, top]).abs() > 1e-4 if top < E else torch.ones(n, dtype=torch.bool)
    assert torch.equal(chosen[clear].sort(-1).values, idx[clear].sort(-1).values) and clear.sum() > 0.9 * n
    assert (weights[clear].double() - val[clear]).abs().max() < 1e-5
    want = plain.experts_ff(mlp, w, "", x.double())
    tol = 2e-5 if dtype == torch.float32 else 0.03
    assert (out.double().cpu()[clear] - want[clear]).abs().max() < tol * float(want.abs().max())
    assert n * top < part.TC_FROM_PAIRS or dtype == torch.float32 or ops.tc_grouped_ok(x.to(DEV), part.w_gu)


def test_the_router_chooses_by_logits_where_sigmoid_scores_all_round_to_one():
    """Logits of 20 to 60 all have a 32-bit sigmoid of exactly 1: the chosen experts are still those of the largest logits, in
    their order, as in the 64-bit statement."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    n, H, E, top = 40, 64, 8, 3
    x = torch.randn(n, H, generator=g)
    w = torch.randn(E, H, generator=g) * 0.2
    w += 40.0 * x[0] / x[0].pow(2).sum()          # every expert's logit for token 0 is near 40
    x[1:] = x[0] + 0.05 * torch.randn(n - 1, H, generator=g)
    z = x.double() @ w.double().T
    assert (torch.sigmoid(z.float()) == 1.0).all() and z.min() > 20
    chosen = torch.empty(n, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(n, top, device=DEV)
    ops.moe_route(x.to(DEV), w.to(DEV), None, chosen, weights, None, scores="sigmoid")
    want = z.topk(top, dim=-1).indices
    gaps = z.sort(-1, descending=True).values
    clear = ((gaps[:, :top] - gaps[:, 1:top + 1]).abs() > 1e-3).all(-1)
    assert clear.sum() > n // 2 and torch.equal(chosen.cpu().long()[clear], want[clear])
    assert (weights.cpu() == 1.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(64, 8, 3, 200), (50, 5, 2, 77), (128, 16, 4, 300)])
def test_the_tokens_own_input(sizes, dtype):
    """Columns [first, first + dim) of the token's table row, gated by gelu_tanh of a projection of x, projected back: the
    part's output before its norm, for few rows and many, against the formula; ids at both ends of the table."""
    from wllm_b200.parts import FEED_FORWARDS, as_branch, spec
    H, dim, layers, vocab = sizes
    g = torch.Generator().manual_seed(H + dim)
    for layer, n in ((0, 5), (layers - 1, 150)):
        w = {"side.embed": torch.randn(vocab, layers * dim, generator=g).to(dtype), f"l{layer}.side.gate": (torch.randn(dim, H, generator=g) * 0.3).to(dtype),
             f"l{layer}.side.proj": (torch.randn(H, dim, generator=g) * 0.3).to(dtype), f"l{layer}.side.norm": torch.ones(H).to(dtype)}
        part = FEED_FORWARDS.build(spec("token_gated_table", table="side.embed", vocab_size=vocab, table_width=layers * dim,
                                        first_column=layer * dim, dim=dim, activation="gelu_tanh", gate_proj=f"l{layer}.side.gate",
                                        out_proj=f"l{layer}.side.proj"), hidden_size=H, model_dtype=dtype)
        part.load(lambda name: w[name].to(DEV))
        tokens = torch.randint(0, vocab, (n,), generator=g)
        tokens[0], tokens[-1] = 0, vocab - 1
        x = torch.randn(n, H, generator=g).to(dtype)
        out = part(x.to(DEV), Scratch(token_ids=tokens.to(torch.int32).to(DEV)))
        got = out.tensor.sum(0) if hasattr(out, "tensor") else out
        wd = {k: v.double() for k, v in w.items()}
        cfg = {"token_side": {"dim": dim}}
        want = plain.token_input(cfg, wd, layer, x.double(), tokens, 1e-6)
        got = plain.rms(got.double().cpu(), 1e-6)
        assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.03) * float(want.abs().max())
