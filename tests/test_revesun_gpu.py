"""Revesun on the GPU against the plain implementation (``tests/plain/revesun.py``).

First every mechanism alone (its kernel against the plain function of the same name, with inputs made so that a fault
shows: one key that dominates, placed far away, at a page border, just inside and just outside a block or a window),
then whole tiny models with random weights under every way of cutting the work: whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches with slots and pages used again, long decoding across several
block edges, and greedy generation through the package's own entry point and scheduler.
"""

import math

import numpy as np
import pytest
import torch

from tests.helpers import (GREEDY_MARGIN, compare, max_live_tokens, random_tokens, replay, trace_mixed, trace_portions,
                           trace_tail, trace_whole)
from tests.plain import revesun as plain
from tests.revesun_models import TINY_REVESUN

pytestmark = pytest.mark.gpu

REL = {"float32": 2e-5, "bfloat16": 3e-2}


def dev():
    return torch.device("cuda", 0)


# ----------------------------------------------------------------------------- mechanisms alone


@pytest.mark.parametrize("groups,width", [(1, 48), (2, 50), (3, 33), (4, 4096), (1, 12288)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_grouped_norm_alone_and_with_the_addition(groups, width, out_dtype):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(groups * 100 + width)
    x = torch.randn(7, width, generator=g) * 3.0
    update = torch.randn(7, width, generator=g)
    weight = 1.0 + 0.2 * torch.randn(width, generator=g)
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    want = plain.grouped_rms_norm(x.double(), weight.double(), groups, 1e-5)
    out = torch.empty(7, width, dtype=out_dtype, device=dev())
    kernels.group_rms_norm(x.to(dev()), None, weight.to(dev()), groups, 1e-5, out)
    assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol)
    for update_dtype in (torch.float32, torch.bfloat16):
        stream = x.to(dev()).clone()
        upd = update.to(dev(), update_dtype)
        kernels.group_rms_norm(stream, upd, weight.to(dev()), groups, 1e-5, out)
        total = x.double() + upd.cpu().double()
        assert torch.allclose(stream.cpu().double(), total, rtol=1e-6, atol=1e-6)      # the sum stays 32-bit
        assert torch.allclose(out.cpu().double(), plain.grouped_rms_norm(total, weight.double(), groups, 1e-5),
                              rtol=tol, atol=tol)


@pytest.mark.parametrize("width", [5, 72, 257, 12288, 14000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_polynorm_alone(width, dtype):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    z = (torch.randn(5, width, generator=g) * 2.0).to(dtype)
    coefficients = torch.tensor([0.7, -0.4, 0.25, 0.1])
    want = plain.polynorm(z.double(), coefficients.double(), 1e-5)
    out = torch.empty_like(z, device=dev())
    kernels.polynorm(z.to(dev()), coefficients.to(dev()), 1e-5, out)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol)
    inplace = z.to(dev()).clone()
    kernels.polynorm(inplace, coefficients.to(dev()), 1e-5, inplace)
    assert torch.equal(inplace, out)


def _pages_from(k, v, page_size, order):
    """Keys ``[T, G, d]`` and values ``[T, G, dv]`` laid into pages taken in ``order``; the block table row."""
    T, G, d = k.shape
    dv = v.shape[2]
    count = -(-T // page_size)
    storage = torch.full((max(order) + 1, G * page_size * (d + dv)), 7.0, dtype=k.dtype)     # stale data everywhere
    for logical in range(count):
        rows = slice(logical * page_size, min(T, (logical + 1) * page_size))
        n = rows.stop - rows.start
        page = storage[order[logical]]
        keys = page[:G * page_size * d].view(G, page_size, d)
        values = page[G * page_size * d:].view(G, page_size, dv)
        keys[:, :n] = k[rows].transpose(0, 1)
        values[:, :n] = v[rows].transpose(0, 1)
    return storage, torch.tensor([order[:count]], dtype=torch.int32)


def _plain_mask(T, kind, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    if kind == "blocks":
        return plain.block_causal_mask(T, size)
    if kind == "window":
        return (j <= i) & (j > i - size)
    return j <= i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,dv", [(4, 2, 16, 24), (3, 3, 20, 12), (6, 1, 40, 8), (2, 1, 128, 128),
                                                 (8, 2, 64, 32), (6, 2, 32, 16), (5, 1, 8, 8), (2, 1, 16, 320),
                                                 (1, 1, 520, 8)])
@pytest.mark.parametrize("kind,size", [("blocks", 300), ("blocks", 16), ("blocks", 7), ("window", 33), ("causal", 0)])
@pytest.mark.parametrize("sink,gated", [(True, True), (False, False)])
def test_masked_attention_sees_exactly_its_keys(dtype, heads, kv_heads, d, dv, kind, size, sink, gated):
    """One query row at a time dominates through one key: the row's output is that key's value if the mask lets the
    row see it, and not otherwise.  The dominant keys stand at position 0, at a block's first position, one before
    it, at page borders and far away; the rows asked are the last of a block, the first of the next, and the end."""
    from tesseract_b200 import kernels

    T, page = 331, 16
    g = torch.Generator().manual_seed(d * 7 + dv)
    q = torch.randn(T, heads, d, generator=g) * 0.3
    k = torch.randn(T, kv_heads, d, generator=g) * 0.3
    v = torch.randn(T, kv_heads, dv, generator=g)
    gate = torch.randn(T, heads * dv, generator=g)
    unit = lambda n: size if kind == "blocks" else page                                           # noqa: E731
    marks = sorted({0, 15, 16, 17, 31, 32, T - 1 - 299, unit(0) - 1, unit(0), 2 * unit(0) - 1, 2 * unit(0)} & set(range(T)))
    for mark in marks:                      # a key that every later row would put all its weight on
        k[mark] = 0.0
        k[mark, :, 0] = 6.0 + 0.01 * mark
    q[:, :, 0] = 4.0
    q, k, v, gate = (t.to(dtype) for t in (q, k, v, gate))
    scale = 0.5
    want = plain.attention_with_sink(q.double(), k.double(), v.double(), scale, _plain_mask(T, kind, size)) \
        if sink else None
    if not sink:                            # the plain function's denominator without the extra entry
        mask = _plain_mask(T, kind, size)
        want = torch.zeros(T, heads, dv, dtype=torch.float64)
        for h in range(heads):
            s = (q[:, h].double() @ k[:, h // (heads // kv_heads)].double().T) * scale
            w = torch.softmax(s.masked_fill(~mask, -math.inf), dim=1)
            want[:, h] = w @ v[:, h // (heads // kv_heads)].double()
    want = want.reshape(T, heads * dv)
    if gated:
        want = want * torch.sigmoid(gate.double())
    order = list(range(40, 40 - (-(-T // page)), -1))                 # pages in descending order, none of them 0
    storage, table = _pages_from(k, v, page, order)
    out = torch.empty(T, heads * dv, dtype=dtype, device=dev())
    positions = torch.arange(T, dtype=torch.int32, device=dev())
    kernels.attention_masked(q.reshape(T, heads * d).to(dev()), gate.to(dev()) if gated else None, out,
                             storage.to(dev()), positions, torch.zeros(T, dtype=torch.int32, device=dev()),
                             table.to(dev()), heads=heads, kv_heads=kv_heads, dim=d, vdim=dv, page_size=page,
                             mask_kind={"causal": 0, "window": 1, "blocks": 2}[kind], mask_size=size, sink=sink,
                             scale=scale)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    got = out.cpu().double()
    bad = (got - want).abs().amax(dim=1) > tol * (1.0 + want.abs().amax(dim=1))
    assert not bad.any(), f"first wrong row {int(bad.nonzero()[0])}"
    # decoded rows: the same rows asked one at a time, out of order, as a batch of single-row sequences
    rows = [T - 1, 16, 15, 0, min(T - 1, unit(0)), max(0, unit(0) - 1)]
    pos = torch.tensor(rows, dtype=torch.int32, device=dev())
    one = torch.empty(len(rows), heads * dv, dtype=dtype, device=dev())
    kernels.attention_masked(q.reshape(T, heads * d)[rows].to(dev()), gate[rows].to(dev()) if gated else None, one,
                             storage.to(dev()), pos, torch.arange(len(rows), dtype=torch.int32, device=dev()),
                             table.repeat(len(rows), 1).to(dev()), heads=heads, kv_heads=kv_heads, dim=d, vdim=dv,
                             page_size=page, mask_kind={"causal": 0, "window": 1, "blocks": 2}[kind], mask_size=size,
                             sink=sink, scale=scale)
    # (a step of few rows shares each row's keys between warps: the same sums in another order)
    assert torch.allclose(one.float(), out[rows].float(), rtol=tol, atol=tol), "a row's result must not depend on its batch"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,heads,kv_heads,d,dv,rot", [(4, 2, 1, 16, 24, 8), (2, 3, 3, 10, 6, 10), (1, 2, 2, 8, 8, 2),
                                                         (3, 1, 1, 7, 5, 4)])
def test_convolution_rotation_and_cache_write(dtype, taps, heads, kv_heads, d, dv, rot):
    """Two sequences in portions (3 + 1 + 2 + 9 rows and 1 + 1 + 20), against the plain convolution and rotation of
    the whole sequences: the state carries the last rows across the cuts, the pages receive every key and value."""
    from tesseract_b200 import kernels

    page, base = 16, 50.0
    channels = heads * d + kv_heads * (d + dv)
    g = torch.Generator().manual_seed(taps * 31 + d)
    lengths = {0: [3, 1, 2, 9], 1: [1, 1, 20]}
    u = {s: (torch.randn(sum(n), channels + 5, generator=g)).to(dtype) for s, n in lengths.items()}
    w = torch.randn(channels, taps, generator=g)
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float()
    state = torch.zeros(4, taps - 1, channels, device=dev()) if taps > 1 else None
    slots = {0: 2, 1: 0}
    storage = torch.zeros(9, kv_heads * page * (d + dv), dtype=dtype, device=dev())
    tables = torch.tensor([[3, 5, 0, 0], [8, 1, 0, 0]], dtype=torch.int32)
    done = {0: 0, 1: 0}
    got_q = {0: [], 1: []}
    for step in range(4):
        seqs = [s for s in (0, 1) if step < len(lengths[s])]
        new = [lengths[s][step] for s in seqs]
        rows = sum(new)
        proj = torch.cat([u[s][done[s]:done[s] + n] for s, n in zip(seqs, new)]).to(dev())
        positions = torch.cat([torch.arange(done[s], done[s] + n) for s, n in zip(seqs, new)]).int().to(dev())
        seq_of_row = torch.cat([torch.full((n,), i) for i, n in enumerate(new)]).int().to(dev())
        row_start = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32, device=dev())
        begin = torch.tensor([done[s] for s in seqs], dtype=torch.int32, device=dev())
        slot = torch.tensor([slots[s] for s in seqs], dtype=torch.int32, device=dev())
        q = torch.empty(rows, heads * d, dtype=dtype, device=dev())
        kernels.conv_rope_cache(proj, w.t().contiguous().to(dev()), state, q, storage, positions, seq_of_row, row_start, begin, slot,
                                tables[seqs].to(dev()), inv_freq.to(dev()), num_seqs=len(seqs), heads=heads,
                                kv_heads=kv_heads, dim=d, vdim=dv, rot_dims=rot, page_size=page, write_kv=True,
                                single=max(new) == 1)
        at = 0
        for s, n in zip(seqs, new):
            got_q[s].append(q[at:at + n].cpu())
            at += n
            done[s] += n
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for s in (0, 1):
        T = sum(lengths[s])
        y = plain.short_convolution(u[s][:, :channels].double(), w.double())
        want_q = plain.rotate_pairs(y[:, :heads * d].reshape(T, heads, d), range(T), rot, base).reshape(T, heads * d)
        want_k = plain.rotate_pairs(y[:, heads * d:heads * d + kv_heads * d].reshape(T, kv_heads, d), range(T), rot, base)
        want_v = y[:, heads * d + kv_heads * d:].reshape(T, kv_heads, dv)
        assert torch.allclose(torch.cat(got_q[s]).double(), want_q, rtol=tol, atol=tol), f"queries of sequence {s}"
        for t in range(T):
            stored = storage[int(tables[s, t // page])].cpu().double()
            keys = stored[:kv_heads * page * d].view(kv_heads, page, d)[:, t % page]
            values = stored[kv_heads * page * d:].view(kv_heads, page, dv)[:, t % page]
            assert torch.allclose(keys, want_k[t], rtol=tol, atol=tol), f"key {t} of sequence {s}"
            assert torch.allclose(values, want_v[t], rtol=tol, atol=tol), f"value {t} of sequence {s}"


@pytest.mark.parametrize("width", [33, 224])
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16)])
def test_gated_recurrence_carries_its_state(width, in_dtype, out_dtype):
    """Three sequences in unequal portions (one of 300 rows, which the kernel cuts into runs; single rows; a slot that
    a finished sequence leaves and a new one takes, zeroed) against the plain walk over the whole sequences."""
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    lengths = {"a": [300, 1, 1, 40], "b": [2, 17, 1, 1], "c": [1, 5]}
    total = {s: sum(n) for s, n in lengths.items()}
    pre = {s: torch.randn(total[s], 3 * width, generator=g) * 2.0 for s in lengths}
    bz, bx = torch.randn(width, generator=g), torch.randn(width, generator=g)
    state = torch.full((3, width), 5.0, device=dev())
    state[:2] = 0.0                                     # slots 0 and 1 start empty; slot 2 is never used
    plan = [(["a", "b"], [0, 1]), (["a", "b"], [0, 1]), (["b", "a"], [1, 0]), (["a", "b"], [0, 1]), (["c"], [1]), (["c"], [1])]
    done = {s: 0 for s in lengths}
    step_of = {s: 0 for s in lengths}
    got = {s: [] for s in lengths}
    for seqs, slot_ids in plan:
        if seqs == ["c"] and step_of["c"] == 0:
            state[1].zero_()                            # what admission does with a slot that is used again
        new = [lengths[s][step_of[s]] for s in seqs]
        proj = torch.cat([pre[s][done[s]:done[s] + n] for s, n in zip(seqs, new)]).to(dev(), in_dtype)
        out = torch.empty(sum(new), width, dtype=out_dtype, device=dev())
        kernels.gated_recurrence(proj, bz.to(dev()), bx.to(dev()), state, out,
                                 torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32, device=dev()),
                                 torch.tensor(slot_ids, dtype=torch.int32, device=dev()), num_seqs=len(seqs),
                                 max_new=max(new))
        at = 0
        for s, n in zip(seqs, new):
            got[s].append(out[at:at + n].cpu())
            at += n
            done[s] += n
            step_of[s] += 1
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    for s in lengths:
        p = pre[s].double()
        z = torch.sigmoid(p[:, :width] + bz.double())
        cand = plain.mingru_candidate(p[:, width:2 * width] + bx.double())
        gate = p[:, 2 * width:]
        S = torch.zeros(width, dtype=torch.float64)
        rows = []
        for t in range(total[s]):
            S = (1 - z[t]) * S + z[t] * cand[t]
            rows.append(S * gate[t] * torch.sigmoid(gate[t]))
        want = torch.stack(rows)
        assert torch.allclose(torch.cat(got[s]).double(), want, rtol=tol, atol=tol), f"sequence {s}"
    assert torch.all(state[2] == 5.0), "a slot that no sequence of the batch owns must stay as it was"


# ----------------------------------------------------------------------------- whole models


LENGTHS = {"p": [1, 2, 3, 14, 40, 97], "q": [5, 33, 66, 130], "r": [4, 27, 81], "s": [1, 9, 70]}


def make_requests(name):
    vocab = TINY_REVESUN[name]["vocab"]
    return {f"{name}{i}": random_tokens(vocab, n, seed=300 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tesseract_b200.weights.random_init import write_random_model

    made = {}

    def get(name):
        if name not in made:
            made[name] = write_random_model(str(tmp_path_factory.mktemp(f"revesun_{name}")), TINY_REVESUN[name], seed=11)
        return made[name]

    return get


@pytest.fixture(scope="module")
def engines(folders):
    from tesseract_b200.engine import load_model, make_stepper

    models = {}

    def get(name, dtype, capacity_tokens=4096, max_requests=8):
        if (name, dtype) not in models:
            models[(name, dtype)] = load_model(folders(name), dtype=dtype)
        return make_stepper(models[(name, dtype)], capacity_tokens=capacity_tokens, max_requests=max_requests)

    return get


@pytest.fixture(scope="module")
def plains(folders):
    known = {}

    def get(name, requests=None):
        requests = requests if requests is not None else make_requests(name)
        config, tensors = plain.load_folder(folders(name))
        out = {}
        for rid, tokens in requests.items():
            if (name, rid) not in known:
                known[(name, rid)] = plain.forward(config, tensors, tokens).numpy()
            out[rid] = known[(name, rid)]
        return out

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["p", "q", "r", "s"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "twos"])
def test_cuts_match_plain(engines, plains, name, dtype, cut):
    """Whole prompts, prompts with a decoded tail (which crosses block edges), portions of changing size, and portions
    of two and three tokens throughout."""
    requests = make_requests(name)
    if cut == "twos":
        steps = trace_portions(requests, sizes=(2, 3, 2, 2))
    else:
        steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    compare(replay(stepper, steps), plains(name), REL[dtype], f"{name}/{dtype}/{cut}")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_without_pages_in_mixed_batches_and_generation(engines, plains, folders, dtype):
    from tesseract_b200 import LLM, SamplingParams

    requests = make_requests("s")
    requests.update({f"sx{i}": random_tokens(TINY_REVESUN["s"]["vocab"], n, seed=40 + i) for i, n in enumerate([31, 12, 50])})
    steps = trace_mixed(requests, seed=9, live_max=3)
    stepper = engines("s", dtype, capacity_tokens=max_live_tokens(steps), max_requests=3)
    compare(replay(stepper, steps), plains("s", requests), REL[dtype], f"s/{dtype}/mixed")
    llm = LLM(folders("s"), dtype=dtype, kv_capacity_tokens=256, max_running=2, prefill_chunk_tokens=32)
    outs = llm.generate([[1, 2, 3], [4] * 40], SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))
    assert [len(o.token_ids) for o in outs] == [5, 5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["p", "q", "r"])
def test_mixed_batches_with_slots_and_pages_used_again(engines, plains, name, dtype):
    requests = make_requests(name)
    requests.update({f"{name}x{i}": random_tokens(TINY_REVESUN[name]["vocab"], n, seed=17 + i)
                     for i, n in enumerate([50, 21, 90, 34, 7])})
    steps = trace_mixed(requests, seed=5, live_max=3)
    assert max(len(e) for e, _ in steps) >= 3, "the trace should batch several requests"
    stepper = engines(name, dtype, capacity_tokens=max_live_tokens(steps), max_requests=3)
    compare(replay(stepper, steps), plains(name, requests), REL[dtype], f"{name}/{dtype}/mixed")
    assert stepper.cache.pages_reused > 0, "the pool was sized so that pages must be used again"
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_gives_each_request_what_it_gets_alone(engines, dtype):
    """Unequal requests side by side, bit for bit against each alone, in portions that cut blocks and pages."""
    name = "q"
    requests = make_requests(name)
    alone = replay(engines(name, dtype), trace_portions(requests, sizes=(9, 2, 30, 5)))
    together = {}
    stepper = engines(name, dtype)
    from tesseract_b200.engine import StepEntry

    at = {rid: 0 for rid in requests}
    for rid in requests:
        assert stepper.cache.admit(rid)
    sizes = {rid: [9, 2, 30, 5] for rid in requests}
    turn = 0
    while any(at[rid] < len(t) for rid, t in requests.items()):
        batch, meta = [], []
        for rid, tokens in requests.items():
            if at[rid] >= len(tokens):
                continue
            size = sizes[rid][turn % 4]
            if len(tokens) - at[rid] - size == 1:
                size += 1
            part = tokens[at[rid]:at[rid] + size]
            batch.append(StepEntry(rid, part, list(range(len(part)))))
            meta.append((rid, at[rid], len(part)))
            at[rid] += len(part)
        rows = stepper.step(batch).float().cpu().numpy()
        r = 0
        for rid, base, n in meta:
            for place in range(n):
                together[(rid, base + place)] = rows[r]
                r += 1
        turn += 1
    worst = max(float(np.abs(together[key] - alone[key]).max()) for key in alone)
    scale = max(float(np.abs(row).max()) for row in alone.values())
    # the products of a batch take other kernels at other row counts: equal up to rounding, not bit for bit
    assert worst <= REL[dtype] * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_many_block_edges(engines, plains, dtype):
    name = "p"
    tokens = random_tokens(TINY_REVESUN[name]["vocab"], 180, seed=77)
    requests = {"long": tokens}
    steps = trace_tail(requests, tail=170)          # ten tokens of prompt, then 170 decoded one by one
    stepper = engines(name, dtype, capacity_tokens=192)
    compare(replay(stepper, steps), plains(name, requests), REL[dtype], f"{name}/{dtype}/long decode")
    assert stepper.cache.used_pages() == 0


def test_pages_of_finished_blocks_go_back_while_the_request_lives(engines):
    """Block size 13 with pages of 16: by position 100 only the pages of the current block are held."""
    stepper = engines("p", "float32", capacity_tokens=64)     # four pages: less than the request's 100 tokens
    from tesseract_b200.engine import StepEntry

    assert stepper.cache.admit("one")
    tokens = random_tokens(TINY_REVESUN["p"]["vocab"], 100, seed=5)
    for at in range(0, 100, 10):
        stepper.step([StepEntry("one", tokens[at:at + 10], [9])])
        assert stepper.cache.used_pages() <= 3 * sum(1 for g in stepper.cache.groups if g.pool is not None)
    stepper.cache.release("one")
    stepper.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["p", "r"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype, graphs):
    from tesseract_b200 import LLM, SamplingParams

    config, tensors = plain.load_folder(folders(name))
    prompts = [random_tokens(config["vocab"], n, seed=n) for n in (3, 19, 75, 1)]
    steps = 24
    llm = LLM(folders(name), dtype=dtype, kv_capacity_tokens=1024, max_running=3, prefill_chunk_tokens=32,
              cuda_graphs=graphs)
    outs = llm.generate(prompts, SamplingParams(max_tokens=steps, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == steps and out.finish_reason == "length"
        tokens = list(prompt)
        for k, got in enumerate(out.token_ids):
            logits = plain.forward(config, tensors, tokens)[-1].numpy()
            best = int(np.argmax(logits))
            margin = float(logits[best] - logits[got])
            limit = GREEDY_MARGIN[dtype] * float(np.abs(logits).max())
            assert got == best or margin <= limit, f"{name}/{dtype}: token {k} is {got}, plain says {best}"
            tokens.append(got)
    assert llm.stepper.cache.used_pages() == 0
    if graphs:      # decode steps and full prompt portions were replayed as graphs, not issued launch by launch
        assert llm.stepper.graphs.safe and llm.stepper.graphs.replays >= steps - 2
        assert llm.stepper.chunk_graphs.replays >= 1
    del llm
    torch.cuda.empty_cache()


def test_replay_program_runs_a_revesun_folder(folders, tmp_path):
    """``bin/trace_run`` picks the model class by ``config.json`` and writes the logits of the wanted places."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config, tensors = plain.load_folder(folders("r"))
    tokens = random_tokens(config["vocab"], 30, seed=9)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": tokens[20:], "want": [9]}], "end": ["a"]})]
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders("r"), "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "64"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want = plain.forward(config, tensors, tokens).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    second = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    scale = float(np.abs(want).max())
    assert np.abs(first - want[[0, 19]]).max() <= 2e-5 * scale
    assert np.abs(second - want[[29]]).max() <= 2e-5 * scale


def test_command_line_generates_and_prints_the_plan(folders):
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders("p")
    common = [sys.executable, os.path.join(root, "bin", "tesseract"), "--model-path", folder, "--kv-capacity-tokens",
              "256", "--max-running", "2", "--dtype", "float32"]
    done = subprocess.run(common + ["--prompt-ids", "5,6,7,8", "--random-prompt", "11", "--max-tokens", "4",
                                    "--temperature", "0", "--ignore-eos", "--json", "--check-weights"],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert "weights checked: final.norm" in done.stderr
    records = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert len(records) == 2 and all(len(r["token_ids"]) == 4 and r["finish_reason"] == "length" for r in records)
    config, tensors = plain.load_folder(folder)
    tokens = [5, 6, 7, 8]
    for got in records[0]["token_ids"]:
        logits = plain.forward(config, tensors, tokens)[-1].numpy()
        best = int(np.argmax(logits))
        assert got == best or float(logits[best] - logits[got]) <= GREEDY_MARGIN["float32"] * float(np.abs(logits).max())
        tokens.append(got)
    shown = subprocess.run(common + ["--print-plan"], capture_output=True, text=True, timeout=600)
    assert shown.returncode == 0, shown.stderr[-2000:]
    assert "kernel plan for Revesun" in shown.stdout
    assert "mixer 'conv_attention'" in shown.stdout and "mixer 'mingru'" in shown.stdout


@pytest.mark.parametrize("seed", [3, 10, 14, 54, 113, 137])
def test_random_configurations_match_plain_in_float32(tmp_path, seed):
    """Configurations drawn at random (layer kinds, order, every size and constant), each whole, with a decoded tail,
    in portions and in mixed batches.  In 32-bit only: a norm over a group of three numbers magnifies bfloat16's
    rounding without bound, whatever computes it."""
    import random

    from tesseract_b200.engine import load_model, make_stepper
    from tesseract_b200.weights.random_init import write_random_model
    from tests.revesun_models import random_config

    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "model"), config, seed=seed)
    loaded, tensors = plain.load_folder(folder)
    r = random.Random(seed + 1000)
    lengths = [1, r.randint(2, 40), r.randint(41, 140), r.randint(141, 300), r.randint(5, 90)]
    requests = {f"q{i}": random_tokens(config["vocab"], n, seed=seed * 10 + i) for i, n in enumerate(lengths)}
    want = {rid: plain.forward(loaded, tensors, tokens).numpy() for rid, tokens in requests.items()}
    model = load_model(folder, dtype="float32")
    for name, steps in (("whole", trace_whole(requests)), ("tail", trace_tail(requests, tail=20)),
                        ("portions", trace_portions(requests)), ("mixed", trace_mixed(requests, seed=seed, live_max=4))):
        stepper = make_stepper(model, capacity_tokens=max(1024, max_live_tokens(steps)), max_requests=4)
        compare(replay(stepper, steps), want, 3e-5, f"seed {seed}/{name}")
        assert stepper.cache.used_pages() == 0
