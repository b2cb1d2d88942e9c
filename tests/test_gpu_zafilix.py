"""Zafilix on the device against its plain statement (tests/plain_zafilix.py, float64, whole sequences).

Whole models: the residual after every layer run; every way of cutting the work (whole prompts, a tail decoded token by
token, portions down to two tokens and one, mixed batches whose pages are used again), bit for bit against one another in
32-bit; long decoding past every window and block; decoding from captured graphs; greedy generation through the scheduler;
the trace runner.  Mechanisms alone: the norm behind a sublayer with the reader that norms nothing, q and k normed as whole
rows and turned in neighbouring pairs with stretched frequencies, the latent row's norm and turn and the maps of the heads,
attention in blocks and over latent rows in a window (one key made to stand out just inside and just outside every edge,
far back, at page borders, pages in scrambled order, all three kernels), the sigmoid gate, the squared ReLU, the factor and
the cap on the logits.
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zafilix as plain
import traces
from helpers import folder_weights, max_diff
from zafilix_configs import CONFIGS, write_folder

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
    rows' scale: the typical row within 1.5 %, every row within 6 %."""
    assert set(rows) == set(ref)
    scale = max(1.0, max(float(r.abs().max()) for r in ref.values()))
    if dtype == torch.float32:
        assert max_diff(rows, ref) < 2e-4 * scale, what
        return
    rms = math.sqrt(sum(float(r.double().pow(2).mean()) for r in ref.values()) / len(ref))
    rel = sorted(float((rows[k].double() - ref[k].double()).pow(2).mean().sqrt()) / rms for k in ref)
    assert rel[len(rel) // 2] < 0.015 and rel[-1] < 0.06, (what, rel[len(rel) // 2], rel[-1])


def requests_of(name, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in CONFIGS:
        folder = write_folder(str(tmp_path_factory.mktemp("zafilix") / name), name)
        reqs = requests_of(name, (5, 64, 31, 90, 2, 47, 70, 25, 1, 113, 17), seed=3)
        out[name] = (folder, reqs, plain_rows(folder, name, reqs))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_residual_after_every_layer_run(setups, name, dtype):
    """Layer by layer: the residual with each run's last branch folded in, against the plain statement's."""
    from wllm_b200.engine import StepEntry
    folder, reqs, _ = setups[name]
    toks = reqs["r3"]
    w = {k: v.double() for k, v in folder_weights(folder).items()}
    want = plain.layers(CONFIGS[name], w, toks)
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
            got.append((residual.stream + p.norm.branch(p.branch, ctx, "watched_branch")).double().cpu())
    blocks = model.blocks
    model.blocks = [Watched(b) for b in blocks]
    rc = runner.cache.open("x")
    runner.step([StepEntry(rc, toks, [0])])
    model.blocks = blocks
    assert len(got) == len(CONFIGS[name]["layers"])
    for run, (a, b) in enumerate(zip(got, want)):
        tol = (2e-5 if dtype == torch.float32 else 0.03) * float(b.abs().max())
        assert (a - b).abs().max() < tol, (run, float((a - b).abs().max()), tol)


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
        runner = runner_for(folder, dtype, 16, pages)
        rows = traces.run_in_process(runner, steps)
        close_enough(rows, ref, dtype, cut)
        assert all(f == pages for f in runner.cache.free_pages())
        if cut == "mixed":      # pages were used again
            assert all(g.pool.takes > pages for g in runner.cache.groups if g.spec.window is None) and len(reqs) > 4
            assert all(g.pool.takes > 0 for g in runner.cache.groups)
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
def test_long_decoding_passes_every_window_and_block_and_gives_pages_back(setups, name, dtype):
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
        if spec.window is not None:      # a group with a window or blocks holds the pages that its rule still needs, no more
            most = -(-spec.window // 16) + 1
            assert max(h[g] for h in held[40:]) <= most < 15, (spec, held[-1])
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
@pytest.mark.parametrize("H", [40, 50, 256, 1000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_behind_a_sublayer_and_a_reader_that_norms_nothing(H, dtype):
    """x += rms(branch) * (1 + w); the sublayer that follows reads x itself, rounded once to the model's type."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(H)
    n, eps = 7, 1e-5
    x, a = torch.randn(n, H, generator=g) * 3, (torch.randn(n, H, generator=g) * 5).to(dtype)
    w = (torch.randn(H, generator=g) * 0.3).to(dtype)
    want = x.double() + plain.norm_one_plus(a.double(), w.double(), eps)
    resid, out = x.to(DEV), torch.empty(n, H, dtype=dtype, device=DEV)
    ops.sandwich_norm(resid, (a.to(DEV), 0), out, w.to(DEV), False, eps, None, 0.0, False, 0.0, post_offset=1.0)
    assert (resid.cpu().double() - want).abs().max() < 1e-5 * float(want.abs().max())
    assert torch.equal(out.cpu(), resid.cpu().to(dtype))
    # 32-bit partial sums of a product cut along K are added in order first; chosen rows leave the residual as it is
    parts = torch.randn(3, n, H, generator=g)
    want2 = x.double() + plain.norm_one_plus(parts.double().sum(0), w.double(), eps)
    resid2 = x.to(DEV)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    some = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.sandwich_norm(resid2, (parts.to(DEV), 3), some, w.to(DEV), False, eps, None, 0.0, False, 0.0, rows=rows, post_offset=1.0)
    assert torch.equal(resid2.cpu(), x)
    assert (some.cpu().double() - want2[[5, 0]]).abs().max() < (1e-5 if dtype == torch.float32 else 0.01) * float(want2.abs().max())
    # the branch's norm alone (what a model's last layer leaves for the final norm), and the reader without anything pending
    alone = ops.branch_norm((a.to(DEV), 0), w.to(DEV), torch.empty(n, H, device=DEV), eps, offset=1.0)
    assert (alone.cpu().double() - plain.norm_one_plus(a.double(), w.double(), eps)).abs().max() < 1e-5 * 10
    plain_read = ops.rmsnorm(resid, None, None, 0.0, 0.0, torch.empty(n, H, dtype=dtype, device=DEV))
    assert torch.equal(plain_read.cpu(), resid.cpu().to(dtype))


def paged(rows_k, rows_v, page_size, order_seed, spare=3):
    """Keys [L, G, d] (and values [L, G, dv], or None: the values lie inside the keys' rows) of one sequence on pages in
    scrambled order, NaN wherever no token lies: the pools and the block table."""
    L, G, d = rows_k.shape
    pages = -(-L // page_size)
    perm = torch.randperm(pages + spare, generator=torch.Generator().manual_seed(order_seed))[:pages]
    kp = torch.full((pages + spare, G, page_size, d), float("nan"), dtype=rows_k.dtype)
    vp = None if rows_v is None else torch.full((pages + spare, G, page_size, rows_v.shape[-1]), float("nan"), dtype=rows_k.dtype)
    for j in range(L):
        kp[perm[j // page_size], :, j % page_size] = rows_k[j]
        if vp is not None:
            vp[perm[j // page_size], :, j % page_size] = rows_v[j]
    return kp.to(DEV), (None if vp is None else vp.to(DEV)), perm.to(torch.int32)[None].contiguous().to(DEV)


def plain_masked_rows(q, k, v, positions, scale, seen_from):
    """q [n, H, d] at `positions` over keys k [L, G, d] and values v [L, G, dv]; seen_from(p) is the first visible key."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for r, p in enumerate(positions):
        j = torch.arange(k.shape[0])
        seen = (j <= p) & (j >= seen_from(p))
        heads = []
        for a in range(H):
            s = (k[:, a // (H // G)].double() @ q[r, a].double()) * scale
            heads.append(torch.softmax(s.masked_fill(~seen, float("-inf")), 0) @ v[:, a // (H // G)].double())
        out.append(torch.cat(heads))
    return torch.stack(out)


def three_kernels(qd, kp, vp, table, positions, L, H, G, d, dv, ps, window, scale, dtype, in_keys=False):
    """The walk, the split and the tiled kernel on the same rows (one portion of one request), and the last row alone."""
    from wllm_b200.kernels import ops
    n = len(positions)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    req = torch.zeros(n, dtype=torch.int32, device=DEV)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    more = dict(vd=dv, values_in_keys=in_keys)
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
@pytest.mark.parametrize("size", [40, 64, 16, 7, 130, 1, 0])
def test_attention_in_blocks_at_every_edge(size, dtype):
    """One key at a time is made to stand out (along the query, long enough to take all the weight where it is seen): the
    last key of the block before the row's, the first of its own, the row's own position, keys at page and chunk borders and
    key 0 far back.  Rows of a prompt's portion and a single decoded row, pages in scrambled order, all three kernels, whose
    results are one, bit for bit.  Size 0: no mask, every earlier key, a far key among hundreds."""
    g = torch.Generator().manual_seed(size * 7 + 1)
    H, G, d, dv, ps, L = 4, 2, 16, 24, 16, 300
    scale = 0.4
    k, v = torch.randn(L, G, d, generator=g).to(dtype), torch.randn(L, G, dv, generator=g).to(dtype)
    n0 = 236
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, d, generator=g).to(dtype)
    start = (lambda p: p - p % size) if size else (lambda p: 0)
    edges = sorted({e for e in (0, 1, start(n0) - 1, start(n0), start(n0) + 1, n0 - 1, n0, start(L - 1) - 1, start(L - 1), 63, 64, 255, 256, 239, 240)
                    if 0 <= e < L})
    changed = {}
    base = plain_masked_rows(q, k, v, positions, scale, start)
    for edge in edges:
        k2 = k.clone()
        k2[edge] = (q[0, 0::2] * 6).to(dtype)         # along the queries of row n0 (heads 0 and 2: one per key/value head)
        kp2, vp, table = paged(k2, v, ps, 5)
        want = plain_masked_rows(q, k2, v, positions, scale, start)
        outs, last = three_kernels(q.reshape(len(positions), H * d).to(DEV), kp2, vp, table, positions, L, H, G, d, dv, ps, -size, scale, dtype)
        for kind, out in zip(("walk", "split", "tiled"), outs):
            err = (out.double() - want).abs().max()
            assert err < (2e-5 if dtype == torch.float32 else 0.03), (kind, edge, float(err))
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]) and torch.equal(last, outs[0][-1:]), edge
        changed[edge] = float((want[0] - base[0]).abs().max()) > 0.05
    # the key that stands out moves the first row's output when and only when the mask lets it be seen (a row that sees one
    # key gives that key's value whatever its score)
    assert all(changed[e] == (start(n0) <= e <= n0 and start(n0) < n0) for e in edges), changed


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,rank,rot", [(40, 32, 8), (64, 24, 8), (17, 16, 16), (1, 8, 8), (130, 64, 32), (0, 40, 24), (90, 512, 64)])
def test_attention_over_latent_rows_at_every_window_edge(window, rank, rot, dtype):
    """One head of keys for all query heads, the values inside the keys' rows (their first `rank` elements).  The key that
    stands out lies just outside the window, on its first key, at the row itself, at page borders, far back."""
    g = torch.Generator().manual_seed(window * 3 + rank)
    H, ps, L = 3, 16, 300
    row = rank + rot
    scale = 0.3
    k = torch.randn(L, 1, row, generator=g).to(dtype)
    n0 = 236
    positions = list(range(n0, L))
    q = (torch.randn(len(positions), H, row, generator=g) * (4.0 / math.sqrt(row))).to(dtype)
    start = (lambda p: max(0, p - window + 1)) if window else (lambda p: 0)
    edges = sorted({e for e in (0, start(n0) - 1, start(n0), start(n0) + 1, n0, start(L - 1) - 1, start(L - 1), 63, 64, 239, 240, 207, 208)
                    if 0 <= e < L})
    if rank > 256:
        edges = edges[:4] + edges[-2:]
    changed = {}
    base = plain_masked_rows(q, k, k[..., :rank], positions, scale, start)
    for edge in edges:
        k2 = k.clone()
        k2[edge, 0] = (q[0, 1] * 8).to(dtype)
        kp2, _, table = paged(k2, None, ps, 7)
        want = plain_masked_rows(q, k2, k2[..., :rank], positions, scale, start)
        qd = q.reshape(len(positions), H * row).to(DEV)
        if row <= 256:
            outs, last = three_kernels(qd, kp2, kp2, table, positions, L, H, 1, row, rank, ps, window, scale, dtype, in_keys=True)
        else:       # rows longer than the tiled kernel takes: the walk and the split
            from wllm_b200.kernels import ops
            pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
            req = torch.zeros(len(positions), dtype=torch.int32, device=DEV)
            outs = []
            for split in (False, True):
                out = torch.empty(len(positions), H * rank, dtype=dtype, device=DEV)
                chunks = ops.simt_chunks(L, window)
                scratch = torch.empty(len(positions) * H * chunks * (rank + 2), device=DEV) if split else None
                ops.paged_attention_simt(qd, out, kp2, kp2, req, pos_t, table, H, 1, row, ps, window, scale, scratch, chunks, vd=rank, values_in_keys=True)
                outs.append(out.cpu())
            last = outs[0][-1:]
        for out in outs:
            err = (out.double() - want).abs().max()
            assert err < (3e-5 if dtype == torch.float32 else 0.04), (edge, float(err))
        assert all(torch.equal(outs[0], o) for o in outs[1:]) and torch.equal(last, outs[0][-1:]), edge
        changed[edge] = float((want[0] - base[0]).abs().max()) > 0.05
    # the values lie inside the keys' rows: the key that stands out moves the output wherever it is seen, also where it is seen alone
    assert all(changed[e] == (start(n0) <= e <= n0) for e in edges), changed


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,vd,rot,divisor", [(4, 2, 16, 24, 8, 4.0), (3, 3, 32, 32, 32, None), (5, 1, 8, 8, 4, 8.0), (2, 1, 64, 64, 0, None)])
def test_rows_normed_as_wholes_then_turned_in_neighbouring_pairs(nq, nkv, hd, vd, rot, divisor, dtype):
    """q and k are each divided by the root mean square of the token's whole row (all heads), multiplied by a gain of that
    size, then turned: pairs (2i, 2i+1) over the first `rot` elements of every head by position * base^(-2i/rot) / divisor.
    From a single tensor and from 32-bit partial sums; keys and values land in their page slots."""
    from wllm_b200.kernels import ops
    from wllm_b200.parts import spec
    from wllm_b200.parts.base import POSITIONS
    g = torch.Generator().manual_seed(nq * 10 + hd)
    n, ps, eps, base = 9, 4, 1e-5, 300.0
    width = (nq + nkv) * hd + nkv * vd
    positions = torch.tensor([0, 1, 2, 3, 50, 51, 1000, 7, 4095], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 7, 0, 1, 12, 13, 9], dtype=torch.int32)
    rot_cfg = {"dims": rot, "base": base}
    if divisor:
        rot_cfg["scaling"] = {"factor": divisor}
    table = POSITIONS.build(spec("rope", theta=base, head_dim=hd, rotary_dim=rot, exact_table=True, pairing="interleaved",
                                 frequency_divisor=divisor)).inv_freq.to(DEV)
    q_gain, k_gain = (1 + 0.3 * torch.randn(nq * hd, generator=g)).to(dtype), (1 + 0.3 * torch.randn(nkv * hd, generator=g)).to(dtype)
    for parts, pad in ((0, 5), (3, 5), (0, 8)):       # a pitch in steps of 8 elements: the kernel with 16-byte accesses, where the sizes allow
        x = torch.randn(max(parts, 1), n, width + pad, generator=g) * 2
        x = x if parts else x[0].to(dtype)
        whole = (x.double().sum(0) if parts else x.double())
        q = plain.norm_plain(whole[:, :nq * hd], q_gain.double(), eps).view(n, nq, hd)
        k = plain.norm_plain(whole[:, nq * hd:(nq + nkv) * hd], k_gain.double(), eps).view(n, nkv, hd)
        q, k = plain.turn_neighbours(q, positions, rot_cfg), plain.turn_neighbours(k, positions, rot_cfg)
        v = whole[:, (nq + nkv) * hd:width].view(n, nkv, vd)
        kp, vp = torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV), torch.zeros(4, nkv, ps, vd, dtype=dtype, device=DEV)
        q_out = torch.empty(n, nq * hd, dtype=dtype, device=DEV)
        ops.rope_row_norm_kv_write(x.to(DEV), q_out, positions.to(DEV), slots.to(DEV), table, kp, vp, nq, nkv, hd, rot, ps, q_gain.to(DEV),
                                   k_gain.to(DEV), eps, nq * hd, nkv * hd, in_splits=parts, pairing="interleaved", vd=vd)
        tol = 2e-5 if dtype == torch.float32 else 0.04
        # the angle is a 32-bit product: at position 4095 it is rounded to a few 1e-4 of a radian, which the 64-bit statement is not
        turned = max(tol, 3e-4)
        assert (q_out.cpu().double().view(n, nq, hd) - q).abs().max() < turned * float(q.abs().max())
        for t in range(n):
            page, at = int(slots[t]) // ps, int(slots[t]) % ps
            assert (kp[page, :, at].cpu().double() - k[t]).abs().max() < (turned if positions[t] > 100 else tol) * float(k.abs().max())
            assert (vp[page, :, at].cpu().double() - v[t]).abs().max() < tol * float(v.abs().max())
        for page, at in ((0, 2), (0, 3), (2, 0), (2, 2), (2, 3), (3, 2), (3, 3)):                # no other slot was written
            assert float(kp[page, :, at].abs().max()) == 0 and float(vp[page, :, at].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dim,rot,rank,vd", [(4, 16, 8, 32, 12), (3, 10, 6, 20, 6), (2, 24, 16, 40, 16), (2, 128, 64, 512, 128)])
def test_latent_row_queries_and_the_heads_maps(H, dim, rot, rank, vd, dtype):
    """The cache row [rms(latent) * gain | key part turned in halves | zeros], the queries' turned parts behind the columns
    that the keys' map fills, and the two maps of the heads: with them a head's score over the cached row equals the score
    against the key written out, and the mapped output equals the sum over written-out values."""
    from wllm_b200.kernels import ops
    from wllm_b200.parts import spec
    from wllm_b200.parts.base import POSITIONS
    g = torch.Generator().manual_seed(H + dim)
    n, ps, eps, base = 6, 4, 1e-5, 100.0
    row = -(-(rank + rot) // 8) * 8
    width = H * (dim + rot) + rank + rot
    positions = torch.tensor([0, 1, 33, 2, 700, 5], dtype=torch.int32)
    slots = torch.tensor([8, 9, 2, 3, 15, 4], dtype=torch.int32)
    rot_cfg = {"dims": rot, "base": base}
    table = POSITIONS.build(spec("rope", theta=base, head_dim=rot, rotary_dim=rot, exact_table=True, pairing="half")).inv_freq.to(DEV)
    gain = (1 + 0.3 * torch.randn(rank, generator=g)).to(dtype)
    uk, uv = (torch.randn(H * dim, rank, generator=g) * 0.2).to(dtype), (torch.randn(H * vd, rank, generator=g) * 0.2).to(dtype)
    for parts in (0, 2):
        x = torch.randn(max(parts, 1), n, width, generator=g)
        x = x if parts else x[0].to(dtype)
        whole = x.double().sum(0) if parts else x.double()
        q = whole[:, :H * (dim + rot)].view(n, H, dim + rot)
        c = plain.norm_plain(whole[:, H * (dim + rot):H * (dim + rot) + rank], gain.double(), eps)
        t = plain.turn_halves(whole[:, H * (dim + rot) + rank:].view(n, 1, rot), positions, rot_cfg)[:, 0]
        q_turned = plain.turn_halves(q[..., dim:].contiguous(), positions, rot_cfg)
        pages = torch.full((4, 1, ps, row), float("nan"), dtype=dtype, device=DEV)
        q_plain, q_mapped = torch.empty(n, H * dim, dtype=dtype, device=DEV), torch.full((n, H * row), float("nan"), dtype=dtype, device=DEV)
        ops.latent_prepare(x.to(DEV), parts, positions.to(DEV), slots.to(DEV), table, gain.to(DEV), eps, pages, ps, q_plain, q_mapped, H, dim,
                           rot, rot, rank, row, pairing="half")
        w_uk_t = uk.view(H, dim, rank).transpose(1, 2).contiguous().to(DEV)
        ops.head_linear(q_plain.view(n, H, dim), w_uk_t, q_mapped.view(n, H, row)[:, :, :rank])
        tol = 2e-5 if dtype == torch.float32 else 0.04
        cached = torch.stack([pages[int(s) // ps, 0, int(s) % ps] for s in slots]).cpu().double()
        assert (cached[:, :rank] - c).abs().max() < tol * float(c.abs().max())
        # the angle is a 32-bit product: at position 4095 it is rounded to a few 1e-4 of a radian, which the 64-bit statement is not
        assert (cached[:, rank:rank + rot] - t).abs().max() < max(tol, 3e-4) * float(t.abs().max())
        assert float(cached[:, rank + rot:].abs().sum()) == 0 and not torch.isnan(q_mapped).any()
        # scores of every query against every cached row, both ways
        keys = torch.cat([(c @ uk.double().T).view(n, H, dim), t[:, None].expand(n, H, rot)], dim=-1)
        queries = torch.cat([q[..., :dim], q_turned], dim=-1)
        want = torch.einsum("ihd,jhd->hij", queries, keys)
        got = torch.einsum("ihr,jr->hij", q_mapped.view(n, H, row).cpu().double(), cached)
        assert (got - want).abs().max() < (1e-4 if dtype == torch.float32 else 0.06) * float(want.abs().max())
        # the values' map on a weighted sum of latent rows
        p = torch.softmax(torch.randn(n, H, n, generator=g).double(), -1)
        mixed = torch.einsum("ihj,jr->ihr", p, c).to(dtype)
        out = ops.head_linear(mixed.to(DEV), uv.view(H, vd, rank).contiguous().to(DEV), torch.empty(n, H, vd, dtype=dtype, device=DEV))
        want_v = torch.einsum("ihj,jhv->ihv", p, (c @ uv.double().T).view(n, H, vd))
        assert (out.cpu().double() - want_v).abs().max() < (1e-5 if dtype == torch.float32 else 0.03) * max(1.0, float(want_v.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,K,N", [(3, 16, 40), (2, 40, 24), (5, 10, 6), (4, 128, 512)])
def test_heads_maps_at_every_step_size(H, K, N, dtype):
    """y[t, h] = W_h x[t, h] from one token to hundreds (bfloat16 takes a kernel of its own for few tokens and a batched
    product for many), x read in place from rows that hold more than x, y written into rows that hold more than y; a token's
    result is the same, bit for bit, alone and among others of a step of the same kind."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 100 + K)
    w = (torch.randn(H, N, K, generator=g) * 0.2).to(dtype)
    for n in (1, 8, 9, 31, 32, 200):
        rows = (torch.randn(n, H * (K + 8) + 16, generator=g)).to(dtype)
        x = rows[:, :H * (K + 8)].unflatten(1, (H, K + 8))[:, :, :K]
        want = torch.einsum("thk,hjk->thj", x.double(), w.double())
        held = torch.full((n, H, N + 8), float("nan"), dtype=dtype, device=DEV)
        xd = rows.to(DEV)[:, :H * (K + 8)].unflatten(1, (H, K + 8))[:, :, :K]
        ops.head_linear(xd, w.to(DEV), held[:, :, :N])
        got = held[:, :, :N].cpu()
        assert torch.isnan(held[:, :, N:]).all() and not torch.isnan(got).any()
        tol = 2e-5 if dtype == torch.float32 else 0.02
        assert (got.double() - want).abs().max() < tol * max(1.0, float(want.abs().max())), n
        if n in (9, 31):       # the first token alone: the same bits (steps of the same kind)
            alone = torch.empty(1, H, N, dtype=dtype, device=DEV)
            ops.head_linear(xd[:1], w.to(DEV), alone)
            assert torch.equal(alone.cpu(), got[:1]), n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_gate_squared_relu_and_the_logits_factor_and_cap(dtype):
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    n, c = 9, 40
    for parts in (0, 3):
        fused = torch.randn(max(parts, 1), n, 70 + c, generator=g) * 2
        fused = fused if parts else fused[0].to(dtype)
        gate = (fused.double().sum(0) if parts else fused.double())[:, 70:]
        x = torch.randn(n, c, generator=g).to(dtype)
        got = ops.sigmoid_gate(x.to(DEV).clone(), fused.to(DEV), parts, 70)
        assert (got.cpu().double() - x.double() * torch.sigmoid(gate)).abs().max() < (1e-6 if dtype == torch.float32 else 0.02)
    h = (torch.randn(n, 56, generator=g) * 2).to(dtype)
    sq = ops.unit_act(h.to(DEV), torch.empty(n, 56, dtype=dtype, device=DEV), "relu_squared")
    want = torch.relu(h.double()) ** 2
    assert ((sq.cpu().double() - want).abs() / want.clamp(min=1.0)).max() < (1e-5 if dtype == torch.float32 else 0.01) and float(want.max()) > 4
    # the product with the activation on its 32-bit sums (bfloat16: in the tensor-memory product's epilogue)
    a, w = (torch.randn(200, 256, generator=g)).to(dtype), (torch.randn(384, 256, generator=g) * 0.1).to(dtype)
    out = ops.unit_linear(a.to(DEV), w.to(DEV), "relu_squared", torch.empty(200, 384, dtype=dtype, device=DEV),
                          lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    want = torch.relu(a.double() @ w.double().T) ** 2
    assert (out.cpu().double() - want).abs().max() < (1e-4 if dtype == torch.float32 else 0.02) * float(want.max())
    assert ops.tc_gemm_status(DEV) == 0
    if dtype == torch.float32:
        x = torch.randn(7, 33, generator=g) * 40
        capped = ops.tanh_cap(x.to(DEV).clone(), 11.0, 0.25)
        assert (capped.cpu().double() - 11.0 * torch.tanh(x.double() * 0.25 / 11.0)).abs().max() < 1e-5
        assert (ops.scale_rows(x.to(DEV).clone(), 0.3).cpu().double() - x.double() * 0.3).abs().max() < 1e-5


@pytest.mark.parametrize("hd,n0", [(32, 236), (48, 236), (64, 236), (64, 150), (128, 236), (128, 90), (256, 200)])
@pytest.mark.parametrize("size", [40, 64, 16, 7, 130, 100, 1])
def test_tensor_core_attention_in_blocks(size, hd, n0):
    """The bfloat16 kernels (mma.sync; tcgen05 on one CTA a tile of 128 rows and on pairs of CTAs) with a mask of blocks: a
    prompt's portion whose tiles of rows span borders of blocks, and decoded rows of three requests with their keys cut into
    several splits; one key stands out at every edge; pages in scrambled order, of 16 and 64 tokens."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(size * 7 + hd)
    H, G, L, dtype = 4, 2, 300, torch.bfloat16
    scale = 0.4 * (16 / hd) ** 0.5
    k, v = torch.randn(L, G, hd, generator=g).to(dtype), torch.randn(L, G, hd, generator=g).to(dtype)
    positions = list(range(n0, L))
    q = torch.randn(len(positions), H, hd, generator=g).to(dtype)
    start = lambda p: p - p % size
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    edges = sorted({e for e in (0, start(n0) - 1, start(n0), n0, start(L - 1) - 1, start(L - 1), start(L - 3), 63, 64, 127, 128, 255, 256)
                    if 0 <= e < L})
    base = plain_masked_rows(q, k, v, positions, scale, start)
    for ps in (16, 64):
        for edge in edges:
            k2 = k.clone()
            k2[edge] = (q[0, 0::2] * 6).to(dtype)
            kp, vp, table = paged(k2, v, ps, 5 + ps)
            want = plain_masked_rows(q, k2, v, positions, scale, start)
            assert (float((want[0] - base[0]).abs().max()) > 0.05) == (start(n0) <= edge <= n0 and start(n0) < n0)
            qd = q.reshape(len(positions), H * hd).to(DEV)
            out = torch.empty(len(positions), H * hd, dtype=dtype, device=DEV)
            ops.attention_mma_prefill(qd, out, kp, vp, one(0), one(len(positions)), one(L), table, len(positions), H, G, hd, ps, -size,
                                      scale, skip_single=False)
            err = (out.cpu().double() - want).abs().max()
            assert err < 0.03, ("prefill", ps, edge, float(err))
            R = 3
            tables = table.expand(R, -1).contiguous()
            starts, lens = torch.arange(R, dtype=torch.int32, device=DEV), torch.ones(R, dtype=torch.int32, device=DEV)
            ctxs = torch.tensor([L - 2, L - 1, L], dtype=torch.int32, device=DEV)
            for split_keys, max_splits in ((512, 1), (128, 3), (64, 5)):
                scratch = torch.empty(ops.attention_mma_scratch_floats(R, H, hd, max_splits), device=DEV)
                od = torch.empty(R, H * hd, dtype=dtype, device=DEV)
                ops.attention_mma_decode(qd[-3:].contiguous(), od, kp, vp, starts, lens, ctxs, tables, H, G, hd, ps, -size, scale,
                                         split_keys, max_splits, scratch)
                err = (od.cpu().double() - want[-3:]).abs().max()
                assert err < 0.03, ("decode", ps, edge, split_keys, float(err))
    assert ops.tc_gemm_status(DEV) == 0


@pytest.mark.parametrize("window,rank,rot,H", [(40, 32, 8, 3), (64, 96, 32, 4), (17, 64, 16, 5), (1, 32, 8, 2), (130, 160, 48, 6), (0, 64, 24, 3),
                                               (90, 512, 64, 16), (33, 256, 40, 1), (-48, 64, 8, 3)])
def test_tensor_core_attention_over_latent_rows(window, rank, rot, H):
    """The bfloat16 kernel that takes 64 (token, head) rows of a request a CTA: in one launch the last tokens of one sequence
    (tiles of rows that span the window's edge), a whole short prompt and a single decoded token, each sequence on pages of
    its own in scrambled order, pages of 16 and 64 tokens.  One key stands out at every edge.  A negative window is a mask of
    blocks."""
    from wllm_b200.kernels import ops
    g = torch.Generator().manual_seed(abs(window) * 3 + rank)
    L, n0, dtype = 300, 236, torch.bfloat16
    row = rank + rot
    scale = 0.3
    assert ops.latent_mma_ok(H, rank, row, 16)
    k = torch.randn(L, 1, row, generator=g).to(dtype)
    positions = list(range(n0, L))
    q = (torch.randn(len(positions), H, row, generator=g) * (4.0 / math.sqrt(row))).to(dtype)
    if window > 0:
        start = lambda p: max(0, p - window + 1)
    elif window < 0:
        start = lambda p: p - p % (-window)
    else:
        start = lambda p: 0
    edges = sorted({e for e in (0, start(n0) - 1, start(n0), start(n0) + 1, n0, start(L - 1) - 1, start(L - 1), 31, 32, 63, 64, 255, 256)
                    if 0 <= e < L})
    if rank > 128:
        edges = edges[:3] + edges[-2:]
    # two more requests beside the portion: a whole prompt of 70 tokens and a sequence of 150 that brings its last token
    short_k, long_k = torch.randn(70, 1, row, generator=g).to(dtype), torch.randn(150, 1, row, generator=g).to(dtype)
    short_q = (torch.randn(70, H, row, generator=g) * (4.0 / math.sqrt(row))).to(dtype)
    long_q = (torch.randn(1, H, row, generator=g) * (4.0 / math.sqrt(row))).to(dtype)
    want_short = plain_masked_rows(short_q, short_k, short_k[..., :rank], list(range(70)), scale, start)
    want_long = plain_masked_rows(long_q, long_k, long_k[..., :rank], [149], scale, start)
    base = plain_masked_rows(q, k, k[..., :rank], positions, scale, start)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    for ps in (16, 64):
        for edge in edges:
            k2 = k.clone()
            k2[edge, 0] = (q[0, H // 2] * 8).to(dtype)
            want = plain_masked_rows(q, k2, k2[..., :rank], positions, scale, start)
            assert (float((want[0] - base[0]).abs().max()) > 0.05) == (start(n0) <= edge <= n0)
            pools, tables = [], []
            for rows_k, seed in ((k2, 7), (short_k, 8), (long_k, 9)):
                kp, _, table = paged(rows_k, None, ps, seed + ps)
                tables.append(table[0] + sum(p.shape[0] for p in pools))
                pools.append(kp)
            width = max(t.numel() for t in tables)
            table = torch.stack([torch.nn.functional.pad(t, (0, width - t.numel())) for t in tables]).contiguous()
            pool = torch.cat(pools).contiguous()
            qd = torch.cat([q.reshape(-1, H * row), short_q.reshape(-1, H * row), long_q.reshape(-1, H * row)]).to(DEV)
            out = torch.empty(qd.shape[0], H * rank, dtype=dtype, device=DEV)
            n = len(positions)
            ops.latent_attention_mma(qd, out, pool, i32([0, n, n + 70]), i32([n, 70, 1]), i32([L, 70, 150]), table, 70, H, rank, row, ps,
                                     window, scale)
            got = out.cpu().double()
            for what, a, b in (("portion", got[:n], want), ("whole", got[n:n + 70], want_short), ("single", got[n + 70:], want_long)):
                err = (a - b).abs().max()
                assert err < 0.04, (what, ps, edge, float(err))
            # single tokens alone: the last three positions of the sequence as three requests, their keys whole and in splits
            R = 3
            tables3 = table[:1].expand(R, -1).contiguous()
            for split_tiles in (0, 1, 2, 5):
                tiles = -(-L // 32) if window == 0 else min(-(-L // 32), -(-abs(window) // 32) + 1)
                max_splits = -(-tiles // split_tiles) if split_tiles else 1
                scratch = torch.full((ops.latent_mma_scratch_floats(R, H, rank, max_splits),), float("nan"), device=DEV) if split_tiles else None
                od = torch.empty(R, H * rank, dtype=dtype, device=DEV)
                ops.latent_attention_mma(qd[n - 3:n].contiguous(), od, pool, i32([0, 1, 2]), i32([1, 1, 1]), i32([L - 2, L - 1, L]), tables3, 1,
                                         H, rank, row, ps, window, scale, split_tiles=split_tiles, max_splits=max_splits, scratch=scratch)
                err = (od.cpu().double() - want[-3:]).abs().max()
                assert err < 0.04, ("singles", ps, edge, split_tiles, float(err))
