"""Pekodra on the GPU against the plain implementation (``tests/plain/pekodra.py``).

First every mechanism alone (its kernel or part against the plain function of the same name, with inputs made so that
a fault shows: one key that dominates, placed far away, at a page border, just inside and just outside a window),
then whole tiny models with random weights under every way of cutting the work: whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches with slots and pages used again, long decoding while the window
moves over decoded tokens, and greedy generation through the package's own entry point and scheduler.
"""

import math

import numpy as np
import pytest
import torch

from tests.helpers import (GREEDY_MARGIN, compare, max_live_tokens, random_tokens, replay, trace_mixed, trace_portions,
                           trace_tail, trace_whole)
from tests.pekodra_models import TINY_PEKODRA
from tests.plain import pekodra as plain

pytestmark = pytest.mark.gpu

REL = {"float32": 2e-5, "bfloat16": 3e-2}


def dev():
    return torch.device("cuda", 0)


def runtime(dtype):
    from tesseract_b200.parts import Runtime

    return Runtime(dtype, dev())


# ----------------------------------------------------------------------------- mechanisms alone


@pytest.mark.parametrize("width", [5, 48, 66, 4096, 12288])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_two_norms_of_one_sum(width, out_dtype):
    """The pending sum and two norms with weights stored around zero from one kernel, with no, one and two updates."""
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    x = torch.randn(6, width, generator=g) * 3.0
    a, b = torch.randn(6, width, generator=g), torch.randn(6, width, generator=g) * 2.0
    w1, w2 = 0.2 * torch.randn(width, generator=g), 0.2 * torch.randn(width, generator=g)
    tol = 2e-6 if out_dtype == torch.float32 else 1e-2
    for updates in ((), (a,), (a, b)):
        total = x.double() + (sum(u.double() for u in updates) if updates else 0.0)
        stream = x.to(dev()).clone()
        y1 = torch.empty(6, width, dtype=out_dtype, device=dev())
        y2 = torch.empty_like(y1)
        on_device = [u.to(dev()) for u in updates] + [None, None]
        kernels.sum_norms(stream, on_device[0], on_device[1], (1.0 + w1).to(dev()), y1, (1.0 + w2).to(dev()), y2, 1e-6)
        assert torch.allclose(stream.cpu().double(), total, rtol=1e-6, atol=1e-6)         # the sum stays 32-bit
        assert torch.allclose(y1.cpu().double(), plain.offset_rms_norm(total, w1.double(), 1e-6), rtol=tol, atol=tol)
        assert torch.allclose(y2.cpu().double(), plain.offset_rms_norm(total, w2.double(), 1e-6), rtol=tol, atol=tol)
        alone = torch.empty_like(y1)
        kernels.sum_norms(x.to(dev()).clone(), on_device[0], on_device[1], (1.0 + w2).to(dev()), alone, None, None, 1e-6)
        assert torch.equal(alone, y2)


def test_the_norm_part_adds_one_to_its_stored_weight():
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import NORMS

    g = torch.Generator().manual_seed(1)
    w = (0.3 * torch.randn(40, generator=g)).to(torch.bfloat16)
    x = torch.randn(3, 40, generator=g)
    spec = PartSpec.make("grouped_rms_norm", {"size": 40, "groups": 1, "eps": 1e-5, "offset": 1.0}, {"weight": "w"})
    norm = NORMS.get(spec.kind)(spec, {"weight": w}, runtime(torch.float32))
    want = plain.offset_rms_norm(x.double(), w.double(), 1e-5)
    assert torch.allclose(norm.forward(x.to(dev())).cpu().double(), want, rtol=2e-6, atol=2e-6)
    a, b = torch.randn(3, 40, generator=g), torch.randn(3, 40, generator=g)
    stream = x.to(dev()).clone()
    got = norm.forward_sum(stream, a.to(dev()), b.to(dev()))
    want = plain.offset_rms_norm(x.double() + a.double() + b.double(), w.double(), 1e-5)
    assert torch.allclose(got.cpu().double(), want, rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [7, 64, 1000])
def test_gated_activation_with_biases_and_small_kernels(dtype, inter):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(inter)
    gu = (torch.randn(5, 2 * inter, generator=g) * 2.0).to(dtype)
    bias = torch.randn(2 * inter, generator=g)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for b in (bias, None):
        gate, up = gu[:, :inter].double(), gu[:, inter:].double()
        if b is not None:
            gate, up = gate + b[:inter].double(), up + b[inter:].double()
        out = torch.empty(5, inter, dtype=dtype, device=dev())
        kernels.gated_activation(gu.to(dev()), None if b is None else b.to(dev()), out, kernels.ACT_GELU_TANH)
        assert torch.allclose(out.cpu().double(), plain.gelu_tanh(gate) * up, rtol=tol, atol=tol)
    z = gu.to(dev())
    out = torch.empty_like(z)
    kernels.squared_relu(z, out)
    assert torch.allclose(out.cpu().double(), torch.relu(gu.double()) ** 2, rtol=tol, atol=tol)
    y = gu.to(dev()).clone()
    kernels.add_bias(y, bias.to(dev()))
    assert torch.allclose(y.cpu().double(), gu.double() + bias.double(), rtol=tol, atol=tol)
    logits = torch.randn(3, 50, generator=g)
    assert torch.equal(kernels.scale_rows(logits.to(dev()).clone(), 0.3).cpu(), logits * 0.3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_and_the_scaled_head(dtype):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import EMBEDDINGS, HEADS

    g = torch.Generator().manual_seed(2)
    table = torch.randn(30, 24, generator=g).to(torch.bfloat16)
    spec = PartSpec.make("token_embedding", {"vocab_size": 30, "hidden_size": 24, "stream": "float32", "scale": 2.5},
                         {"table": "t"})
    part = EMBEDDINGS.get(spec.kind)(spec, {"table": table}, runtime(dtype))
    tokens = torch.tensor([3, 29, 0, 3], dtype=torch.int32, device=dev())
    got = part.forward(tokens)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), table.float()[[3, 29, 0, 3]] * 2.5)
    head_spec = PartSpec.make("lm_head", {"vocab_size": 30, "hidden_size": 24, "scale": 0.375}, {"weight": "h"})
    head = HEADS.get(head_spec.kind)(head_spec, {"weight": table}, runtime(dtype))
    x = torch.randn(5, 24, generator=g).to(dtype)
    want = (x.double() @ table.double().T) * 0.375
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(head.forward(x.to(dev())).cpu().double(), want, rtol=tol, atol=tol)


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,dv,rot", [(4, 2, 16, 24, 8), (3, 3, 20, 12, 20), (6, 1, 40, 8, 0),
                                                     (2, 1, 128, 64, 64), (5, 1, 6, 10, 2)])
@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 32, "fast": 16.0, "slow": 1.0}])
def test_rotation_unit_norm_and_page_write(dtype, heads, kv_heads, d, dv, rot, scaling):
    """Rotation of halves with blended frequencies, the division by the head's root mean square and the write into
    pages taken in scrambled order, in two portions of one sequence (the second starts in the middle of a page)."""
    from tesseract_b200 import kernels
    from tesseract_b200.parts.rotary import blended_inverse_frequencies

    T, page, cut = 45, 16, 21
    g = torch.Generator().manual_seed(d + dv)
    proj = torch.randn(T, heads * d + kv_heads * (d + dv) + 3, generator=g).to(dtype)      # three numbers behind are left alone
    freqs, amplitude = blended_inverse_frequencies(rot, 100.0, scaling) if rot else (np.zeros(0), 1.0)
    inv_freq = torch.tensor(np.asarray(freqs, dtype=np.float32), device=dev()) if rot else None
    order = [5, 2, 7]
    storage = torch.full((8, kv_heads * page * (d + dv)), 7.0, dtype=dtype, device=dev())
    table = torch.tensor([order], dtype=torch.int32, device=dev())
    q = torch.empty(T, heads * d, dtype=dtype, device=dev())
    for lo, hi in ((0, cut), (cut, T)):
        positions = torch.arange(lo, hi, dtype=torch.int32, device=dev())
        seq = torch.zeros(hi - lo, dtype=torch.int32, device=dev())
        kernels.rope_norm_cache(proj[lo:hi].to(dev()), q[lo:hi], storage, positions, seq, table, inv_freq,
                                amplitude=amplitude, heads=heads, kv_heads=kv_heads, dim=d, vdim=dv, rot_dims=rot,
                                unit_norm=True, eps=1e-6, page_size=page)
    wide = proj.double()
    want_q = wide[:, :heads * d].reshape(T, heads, d)
    want_k = wide[:, heads * d:(heads + kv_heads) * d].reshape(T, kv_heads, d)
    want_v = wide[:, (heads + kv_heads) * d:(heads + kv_heads) * d + kv_heads * dv].reshape(T, kv_heads, dv)
    if rot:
        plain_freqs, plain_amplitude = plain.blended_frequencies(rot, 100.0, scaling)
        want_q = plain.rotate_half(want_q, range(T), rot, plain_freqs, plain_amplitude)
        want_k = plain.rotate_half(want_k, range(T), rot, plain_freqs, plain_amplitude)
    want_q, want_k = plain.unit_rms(want_q, 1e-6), plain.unit_rms(want_k, 1e-6)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(q.cpu().double().reshape(T, heads, d), want_q, rtol=tol, atol=tol)
    want_pages, _ = _pages_from(want_k, want_v, page, order)
    got = storage.cpu().double()
    for logical, page_id in enumerate(order):
        n = min(page, T - logical * page)
        got_k = got[page_id][:kv_heads * page * d].view(kv_heads, page, d)[:, :n]
        got_v = got[page_id][kv_heads * page * d:].view(kv_heads, page, dv)[:, :n]
        assert torch.allclose(got_k, want_pages[page_id][:kv_heads * page * d].view(kv_heads, page, d)[:, :n], rtol=tol, atol=tol)
        assert torch.equal(got_v, want_pages[page_id][kv_heads * page * d:].view(kv_heads, page, dv)[:, :n])
    untouched = [p for p in range(8) if p not in order]
    assert torch.all(storage[untouched] == 7.0), "pages that the table does not name stay as they were"


def _attention_part(dtype, heads, kv_heads, d, dv, window, scale, tensors, rot=None):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    children = {}
    if rot:
        children["position"] = PartSpec.make("rotary_blend", {"head_dim": d, "dims": rot[0], "base": rot[1],
                                                              "scaling": rot[2]})
    mask = (("kind", "window"), ("size", window)) if window else (("kind", "causal"),)
    spec = PartSpec.make("normed_attention",
                         {"hidden_size": tensors["q"].shape[1], "num_heads": heads, "num_kv_heads": kv_heads,
                          "key_dim": d, "value_dim": dv, "scale": scale, "mask": mask, "qk_norm_eps": 1e-6,
                          "stream": "float32"},
                         {n: n for n in tensors}, children)
    return MIXERS.get(spec.kind)(spec, tensors, runtime(dtype))


def _step_context(positions, page_order, page):
    """A step of one sequence whose rows stand at ``positions`` (consecutive), with the given block table."""
    from tesseract_b200.parts import GroupView, StepContext

    n = len(positions)
    as_i32 = lambda values: torch.tensor(values, dtype=torch.int32, device=dev())         # noqa: E731
    return StepContext(num_rows=n, num_seqs=1, token_ids=as_i32([0] * n), positions=as_i32(list(positions)),
                       seq_of_row=as_i32([0] * n), row_start=as_i32([0, n]), seq_begin=as_i32([positions[0]]),
                       state_slots=as_i32([0]), groups=[GroupView(as_i32([page_order]), page)],
                       host_new=[n], host_begin=[positions[0]], host_slots=[0], max_new=n, max_context=positions[-1] + 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,dv", [(4, 2, 16, 24), (8, 2, 64, 48), (3, 1, 20, 12), (4, 1, 64, 64),
                                                 (2, 2, 128, 128), (2, 1, 64, 128), (2, 1, 128, 64)])
@pytest.mark.parametrize("window", [33, 16, 5, 1, None])
def test_window_attention_sees_exactly_its_keys(dtype, heads, kv_heads, d, dv, window):
    """A row whose query equals one key's direction returns that key's value if the window lets the row see the key,
    and not otherwise.  The mixer's projections are made selectors, so that a row of the input IS its queries, keys
    and values side by side; for chosen (row, key) pairs the row's queries and the key are one strong direction.  The
    dominant keys stand at the window's first position, one before it, at position 0, at page borders and (without a
    window) hundreds of positions back; rows are asked inside a prompt portion and as single decoded rows, with pages
    taken in scrambled order.  That the test is sharp is itself asserted: the plain model with a window one position
    longer or shorter changes some asked row."""
    from tesseract_b200.parts import CacheBinding

    T, page = 331, 16
    scale = 40.0 / d                                   # unit-norm heads: a matching pair scores 40
    q_w, k_w, v_w = heads * d, kv_heads * d, kv_heads * dv
    width = q_w + k_w + v_w
    eye = torch.eye(width)
    g = torch.Generator().manual_seed(window or 99)
    tensors = {"q": eye[:q_w], "k": eye[q_w:q_w + k_w], "v": eye[q_w + k_w:],
               "o": torch.randn(24, heads * dv, generator=g) * (heads * dv) ** -0.5}
    tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    part = _attention_part(dtype, heads, kv_heads, d, dv, window, scale, tensors)
    reach = window if window else T
    rows = [330, 300, 257, 256, 200, 64, 48, 17, reach - 1, reach]
    backs = [reach - 1, reach, 0, 1, 15, 16, reach - 1, reach, reach - 1, reach]
    h = torch.randn(T, width, generator=g)
    directions = {}
    pairs = []
    for row, back in zip(rows, backs):
        key = row - back
        if not (0 <= key <= row < T) or any(row == r for r, _ in pairs):
            continue
        if key not in directions:
            directions[key] = torch.randn(kv_heads, d, generator=g) * 2.0
            h[key, q_w:q_w + k_w] = directions[key].reshape(-1)
        h[row, :q_w] = directions[key].repeat_interleave(heads // kv_heads, dim=0).reshape(-1)
        pairs.append((row, key))
    assert len(pairs) >= 4
    h = h.to(dtype)
    weights = {n: t.double() for n, t in tensors.items()}
    shape = {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": dv, "scale": scale}
    want = plain.window_attention(h.double(), weights, dict(shape, mask={"size": window} if window else None), 1e-6)
    for off_by_one in (reach + 1, reach - 1):
        if 1 <= off_by_one < T:
            other = plain.window_attention(h.double(), weights, dict(shape, mask={"size": off_by_one}), 1e-6)
            moved = [row for row, _ in pairs if (other[row] - want[row]).abs().max() > 0.05]
            assert moved, "no asked row notices a window that is one position off"
    count = -(-T // page)
    torch.manual_seed(3)
    order = [1 + i for i in torch.randperm(count).tolist()]
    need = part.cache_need()
    assert need.window == window
    elements = need.page_shape(page)[0]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for cut in ("prompt", "decode"):
        storage = torch.full((count + 1, elements), 7.0, dtype=dtype, device=dev())
        binding = CacheBinding(group=0, storage=storage, writes=True, page_size=page)
        portions = [(0, T)] if cut == "prompt" else [(0, 10)] + [(p, p + 1) for p in range(10, T)]
        got = torch.cat([part.forward(h[lo:hi].to(dev()), _step_context(range(lo, hi), order, page), binding)
                         for lo, hi in portions]).cpu().double()
        assert torch.isfinite(got).all()
        worst = (got - want).abs().max().item()
        assert worst <= tol * max(1.0, want.abs().max().item()), f"{cut}: {worst}"


@pytest.mark.parametrize("rows", [1, 7, 300])
@pytest.mark.parametrize("experts,top", [(5, 2), (33, 4), (16, 1), (3, 3), (64, 6), (200, 8)])
def test_the_choice_takes_the_largest_and_weighs_the_chosen_alone(rows, experts, top):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(experts + rows)
    logits = torch.randn(rows, experts, generator=g) * 3.0
    logits[0, experts - 1] = logits[0, 0] = 50.0                   # equal logits: the lower index goes first
    values, want_ids = torch.topk(logits.double(), top, dim=-1)
    ids = torch.empty(rows, top, dtype=torch.int32, device=dev())
    weights = torch.empty(rows, top, dtype=torch.float32, device=dev())
    kernels.choose_topk(logits.to(dev()), ids, weights)
    assert ids[0, 0].item() == 0 and (top == 1 or ids[0, 1].item() == experts - 1)
    assert torch.equal(torch.sort(ids.cpu().long(), dim=1).values[1:], torch.sort(want_ids, dim=1).values[1:])
    chosen = torch.gather(logits.double(), 1, ids.cpu().long())
    assert torch.all(chosen[:, :-1] >= chosen[:, 1:]), "largest first"
    assert torch.allclose(weights.cpu().double(), torch.softmax(chosen, dim=-1), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 20, 300])
def test_router_of_the_part_against_plain(dtype, rows):
    part, weights, mlp = _experts_part(dtype, 64, 12, 3, 16, None, seed=rows)
    g = torch.Generator().manual_seed(rows + 1)
    x = torch.randn(rows, 64, generator=g).to(dtype)
    want_ids, want_weights = plain.route(x.double(), weights["router"], 3)
    ids, got = part.route(x.to(dev()))
    assert torch.equal(ids.cpu().long(), want_ids)
    assert torch.allclose(got.cpu().double(), want_weights, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("d,dv", [(64, 64), (64, 48), (128, 128), (64, 128), (128, 64)])
@pytest.mark.parametrize("kind,size", [("window", 100), ("window", 7), ("causal", 0), ("blocks", 90), ("blocks", 16)])
def test_tensor_core_prompt_attention_against_plain_and_the_row_kernel(d, dv, kind, size):
    """Three sequences in one step: a whole prompt of 300 rows, 70 rows that continue a sequence at position 500 (the
    keys before them were stored by earlier steps), and a single row at position 40; pages in scrambled order."""
    from tesseract_b200 import kernels

    heads, kv_heads, page = (4, 2, 16) if d == 64 else (12, 1, 16)   # (twelve query heads on one kv head: both halves of a tile)
    scale = 4.0 / d ** 0.5                                           # sharp softmaxes: the weights matter
    spans = [(0, 300), (500, 70), (40, 1)]                           # (first position, rows) of each sequence's portion
    g = torch.Generator().manual_seed(d + dv + size)
    lengths = [begin + n for begin, n in spans]
    pages_each = [-(-length // page) for length in lengths]
    order = torch.randperm(sum(pages_each), generator=g).tolist()
    table = torch.zeros(3, max(pages_each), dtype=torch.int32)
    storage = torch.full((sum(pages_each) + 1, kv_heads * page * (d + dv)), 7.0, dtype=torch.bfloat16)
    qs, wants, used = [], [], 0
    mask_of = {"window": lambda T: plain.window_mask(T, size), "causal": lambda T: plain.window_mask(T, None),
               "blocks": lambda T: plain.window_mask(T, None) & ((torch.arange(T)[:, None] // size) == (torch.arange(T)[None, :] // size))}
    for s, (begin, n) in enumerate(spans):
        T = lengths[s]
        k = torch.randn(T, kv_heads, d, generator=g).to(torch.bfloat16)
        v = torch.randn(T, kv_heads, dv, generator=g).to(torch.bfloat16)
        q = torch.randn(T, heads, d, generator=g).to(torch.bfloat16)
        mine = [1 + p for p in order[used:used + pages_each[s]]]
        used += pages_each[s]
        laid, _ = _pages_from(k, v, page, mine)
        for page_id in mine:
            storage[page_id] = laid[page_id]
        table[s, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
        seen = mask_of[kind](T)
        out = torch.zeros(T, heads, dv, dtype=torch.float64)
        for h in range(heads):
            scores = (q[:, h].double() @ k[:, h // (heads // kv_heads)].double().T) * scale
            out[:, h] = torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1) @ v[:, h // (heads // kv_heads)].double()
        qs.append(q[begin:].reshape(n, heads * d))
        wants.append(out[begin:].reshape(n, heads * dv))
    q_all, want = torch.cat(qs).to(dev()), torch.cat(wants)
    rows = q_all.shape[0]
    positions = torch.cat([torch.arange(b, b + n) for b, n in spans]).to(torch.int32).to(dev())
    seq_of_row = torch.cat([torch.full((n,), s) for s, (_, n) in enumerate(spans)]).to(torch.int32).to(dev())
    row_start = torch.tensor([0, 300, 370, 371], dtype=torch.int32, device=dev())
    mask_kind = {"causal": kernels.MASK_CAUSAL, "window": kernels.MASK_WINDOW, "blocks": kernels.MASK_BLOCKS}[kind]
    got = torch.empty(rows, heads * dv, dtype=torch.bfloat16, device=dev())
    kernels.attention_prompt_mma(q_all, got, storage.to(dev()), positions, row_start, table.to(dev()), num_seqs=3,
                                 heads=heads, kv_heads=kv_heads, dim=d, vdim=dv, page_size=page, mask_kind=mask_kind,
                                 mask_size=size, scale=scale)
    other = torch.empty_like(got)
    kernels.attention_masked(q_all, None, other, storage.to(dev()), positions, seq_of_row, table.to(dev()), heads=heads,
                             kv_heads=kv_heads, dim=d, vdim=dv, page_size=page, mask_kind=mask_kind, mask_size=size,
                             sink=False, scale=scale)
    single = torch.empty_like(got)                                   # the kernel for steps of few rows takes any rows
    kernels.attention_rows_mma(q_all, single, storage.to(dev()), positions, seq_of_row, table.to(dev()), heads=heads,
                               kv_heads=kv_heads, dim=d, vdim=dv, page_size=page, mask_kind=mask_kind, mask_size=size,
                               scale=scale)
    assert (got.cpu().double() - want).abs().max().item() <= 2e-2          # the output's own rounding to bfloat16
    assert (got.float() - other.float()).abs().max().item() <= 2e-2
    assert (single.cpu().double() - want).abs().max().item() <= 2e-2
    assert ((single.cpu().double() - want).abs() <= 1e-2 * want.abs() + 1e-3).all()
    # the weights are 32-bit: an output far below the largest one keeps its relative accuracy
    assert ((got.cpu().double() - want).abs() <= 1e-2 * want.abs() + 1e-3).all()


def _experts_part(dtype, width, experts, top, size, shared, seed):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import FEED_FORWARDS

    g = torch.Generator().manual_seed(seed)
    plain_weights = {"router": torch.randn(experts, width, generator=g) * 2.0 * width ** -0.5}
    for e in range(experts):
        plain_weights[f"e{e}.up"] = torch.randn(size, width, generator=g) * width ** -0.5
        plain_weights[f"e{e}.down"] = torch.randn(width, size, generator=g) * size ** -0.5
    if shared:
        plain_weights["shared.up"] = torch.randn(shared, width, generator=g) * width ** -0.5
        plain_weights["shared.down"] = torch.randn(width, shared, generator=g) * shared ** -0.5
    plain_weights = {n: t.to(torch.bfloat16) for n, t in plain_weights.items()}
    roles = {"router": "router"}
    for e in range(experts):
        roles[f"up.{e}"], roles[f"down.{e}"] = f"e{e}.up", f"e{e}.down"
    if shared:
        roles.update({"shared_up": "shared.up", "shared_down": "shared.down"})
    spec = PartSpec.make("routed_experts", {"hidden_size": width, "num_experts": experts, "top_k": top,
                                            "expert_size": size, "shared_size": shared, "stream": "float32"}, roles)
    part = FEED_FORWARDS.get(spec.kind)(spec, {role: plain_weights[name] for role, name in roles.items()}, runtime(dtype))
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    return part, {n: t.double() for n, t in plain_weights.items()}, mlp


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,experts,top,size,shared", [(64, 3, 2, 32, 48), (40, 5, 1, 24, None), (96, 12, 3, 64, 160),
                                                           (32, 4, 4, 8, 16), (66, 7, 2, 20, 10), (256, 6, 2, 320, 64)])
@pytest.mark.parametrize("rows", [1, 9, 300])
def test_routed_experts_alone(dtype, width, experts, top, size, shared, rows):
    """Router, grouping, both grouped products and the weighted sum against the plain mixture: single rows, a few,
    and so many that an expert's rows fill several tiles; sizes that do and do not go to the tensor cores."""
    part, weights, mlp = _experts_part(dtype, width, experts, top, size, shared, seed=width + experts)
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, width, generator=g).to(dtype)
    want = plain.expert_mixture(x.double(), weights, mlp)
    got = part.forward(x.to(dev()), None)
    assert got.dtype == torch.float32
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got.cpu().double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    # a row's result does not depend on the rows beside it
    if rows > 1:
        alone = part.forward(x[4:5].to(dev()).contiguous(), None)
        assert (alone.cpu() - got[4:5].cpu()).abs().max().item() <= (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_feed_forward_and_origin_mix_alone(dtype):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import FEED_FORWARDS, INJECTIONS, ResidualStream

    g = torch.Generator().manual_seed(5)
    width, inter, rows = 48, 72, 11
    w = {"gate": torch.randn(inter, width, generator=g) * width ** -0.5, "up": torch.randn(inter, width, generator=g) * width ** -0.5,
         "down": torch.randn(width, inter, generator=g) * inter ** -0.5, "gate.b": torch.randn(inter, generator=g),
         "up.b": torch.randn(inter, generator=g), "down.b": torch.randn(width, generator=g)}
    w = {n: t.to(torch.bfloat16) for n, t in w.items()}
    roles = {"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b", "up_bias": "up.b", "down_bias": "down.b"}
    spec = PartSpec.make("gated_mlp", {"hidden_size": width, "intermediate_size": inter, "activation": "gelu_tanh",
                                       "bias": True, "stream": "float32"}, roles)
    part = FEED_FORWARDS.get(spec.kind)(spec, {role: w[name] for role, name in roles.items()}, runtime(dtype))
    x = torch.randn(rows, width, generator=g).to(dtype)
    want = plain.gated_mlp(x.double(), {n: t.double() for n, t in w.items()})
    got = part.forward(x.to(dev()), None)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert got.dtype == torch.float32
    assert (got.cpu().double() - want).abs().max().item() <= tol * want.abs().max().item()

    mix = (torch.randn(width, 2 * width, generator=g) * width ** -0.5).to(torch.bfloat16)
    spec = PartSpec.make("origin_mix", {"hidden_size": width}, {"weight": "m"})
    inject = INJECTIONS.get(spec.kind)(spec, {"weight": mix}, runtime(dtype))
    stream, a, b, origin = (torch.randn(rows, width, generator=g) for _ in range(4))
    for updates in ((None, None), (a, None), (a, b), (None, b)):
        total = stream.double() + sum(u.double() for u in updates if u is not None)
        want = torch.cat([total, origin.double()], dim=1) @ mix.double().T
        kept = origin.to(dev())
        out = inject.forward(ResidualStream(stream.to(dev()), None if updates[0] is None else updates[0].to(dev()),
                                            update_b=None if updates[1] is None else updates[1].to(dev())), kept, None)
        assert out.update is None and out.update_b is None and out.residual.dtype == torch.float32
        assert (out.residual.cpu().double() - want).abs().max().item() <= tol * want.abs().max().item()
        assert torch.equal(kept.cpu(), origin), "the embedding output is only read"


# ----------------------------------------------------------------------------- whole models


LENGTHS = {"a": [1, 2, 3, 14, 40, 97], "b": [5, 33, 66, 130], "c": [4, 27, 81], "d": [1, 9, 70], "e": [300, 5, 270]}


def make_requests(name):
    vocab = TINY_PEKODRA[name]["vocab"]
    return {f"{name}{i}": random_tokens(vocab, n, seed=300 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tesseract_b200.weights.random_init import write_random_model

    made = {}

    def get(name):
        if name not in made:
            made[name] = write_random_model(str(tmp_path_factory.mktemp(f"pekodra_{name}")), TINY_PEKODRA[name], seed=11)
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


class RecordedRouting:
    """Notes which experts the engine's router chose for every (request, position, run of a layer with experts)
    while a trace is replayed, and gives the plain model those choices.

    In bfloat16 the router's input carries rounding noise, and of two nearly equal logits the engine may find the
    other one larger than the plain model does; the outputs then differ by a whole expert, which no tolerance on
    rounding covers.  So the plain model is run with the engine's choices, and the choices themselves are checked
    apart: they must be the plain model's own wherever its margin is not small."""

    def __init__(self, stepper):
        self.stepper = stepper
        self.chosen = {}            # request -> run -> position -> ids
        self.rows, self.run = [], 0

    def __enter__(self):
        from tesseract_b200.parts.experts import RoutedExperts

        self._route, self._step = RoutedExperts.route, self.stepper.step
        recorder = self

        def route(part, x):
            ids, weights = recorder._route(part, x)
            host = ids.cpu()
            for r, (rid, position) in enumerate(recorder.rows):
                recorder.chosen.setdefault(rid, {}).setdefault(recorder.run, {})[position] = host[r]
            recorder.run += 1
            return ids, weights

        def step(entries):
            cache = recorder.stepper.cache
            recorder.rows = [(e.request, cache.length(e.request) + i) for e in entries for i in range(len(e.tokens))]
            recorder.run = 0
            return recorder._step(entries)

        RoutedExperts.route = route
        self.stepper.step = step
        return self

    def __exit__(self, *exc):
        from tesseract_b200.parts.experts import RoutedExperts

        RoutedExperts.route = self._route
        self.stepper.step = self._step

    def plain_logits(self, folder, requests, noise=None):
        """The plain model's logits under the engine's choices; asserts that the choices are its own but for close calls.
        ``noise`` (a dict) receives, per request, what rounding to bfloat16 alone changes at every position."""
        config, tensors = plain.load_folder(folder)
        out, decisions, differing = {}, 0, 0
        for rid, tokens in requests.items():
            routing = {run: torch.stack([by_position[p] for p in range(len(tokens))])
                       for run, by_position in self.chosen.get(rid, {}).items()}
            report = []
            exact = plain.forward(config, tensors, tokens, routing=routing or None, report=report)
            out[rid] = exact.numpy()
            if noise is not None:
                coarse = plain.forward(config, tensors, tokens, routing=routing or None, round_to=torch.bfloat16)
                noise[rid] = (coarse - exact).abs().max(dim=1).values.numpy()
            for run, (own, margin) in enumerate(report):
                for p in range(len(tokens)):
                    decisions += 1
                    if set(own[p].tolist()) != set(routing[run][p].tolist()):
                        differing += 1
                        assert float(margin[p]) < 0.1, f"request {rid} position {p} run {run}: another expert without a close call"
        assert differing <= max(2, 0.03 * decisions), f"{differing} of {decisions} choices differ"
        return out


def replay_against_plain(stepper, steps, folder, requests, dtype, what, measured_noise=False):
    """Replay a trace and compare every wanted row with the plain model (in bfloat16 under the engine's routing).
    ``measured_noise``: a row may also differ by three times what rounding to bfloat16 alone changes at its position in
    the plain model (drawn configurations have positions where that is ten times the usual)."""
    if dtype == "float32":
        config, tensors = plain.load_folder(folder)
        got = replay(stepper, steps)
        want = {rid: plain.forward(config, tensors, tokens).numpy() for rid, tokens in requests.items()}
        return compare(got, want, REL[dtype], what)
    with RecordedRouting(stepper) as recorded:
        got = replay(stepper, steps)
    noise = {} if measured_noise else None
    want = recorded.plain_logits(folder, requests, noise)
    if not measured_noise:
        return compare(got, want, REL[dtype], what)
    for (rid, position), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        limit = max(REL[dtype] * float(np.abs(want[rid]).max()), 3.0 * float(noise[rid][position]))
        err = float(np.abs(row.astype(np.float64) - want[rid][position]).max())
        assert np.isfinite(row).all() and err <= limit, (f"{what}: first wrong token is request {rid!r} position "
                                                         f"{position}: max |diff| {err:.3e} > {limit:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_every_layer_run_matches_plain(engines, folders, name, dtype):
    """The stream after every run of a layer (a looped layer counts each time) against the plain model's."""
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.parts.block import ParallelBlock

    config, tensors = plain.load_folder(folders(name))
    tokens = random_tokens(config["vocab"], 37, seed=8)
    _, want = plain.forward(config, tensors, tokens, keep_layers=True)
    seen = []
    original = ParallelBlock.forward

    def recording(self, stream, ctx, cache):
        out = original(self, stream, ctx, cache)
        total = out.residual.double()
        for update in (out.update, out.update_b):
            total = total + (update.double() if update is not None else 0.0)
        seen.append(total.cpu())
        return out

    stepper = engines(name, dtype)
    assert stepper.cache.admit("one")
    ParallelBlock.forward = recording
    try:
        stepper.step([StepEntry("one", tokens, [len(tokens) - 1])])
    finally:
        ParallelBlock.forward = original
        stepper.cache.release("one")
    assert len(seen) == want.shape[0] == len(plain.run_order(config))
    tol = 2e-5 if dtype == "float32" else 3e-2
    for run, got in enumerate(seen):
        assert (got - want[run]).abs().max().item() <= tol * want[run].abs().max().item(), f"layer run {run}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "twos"])
def test_cuts_match_plain(engines, folders, name, dtype, cut):
    """Whole prompts, prompts with a decoded tail (over which the windows move), portions of changing size, and
    portions of two and three tokens throughout."""
    requests = make_requests(name)
    if cut == "twos":
        steps = trace_portions(requests, sizes=(2, 3, 2, 2))
    else:
        steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/{cut}")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_mixed_batches_with_slots_and_pages_used_again(engines, folders, name, dtype):
    requests = make_requests(name)
    requests.update({f"{name}x{i}": random_tokens(TINY_PEKODRA[name]["vocab"], n, seed=17 + i)
                     for i, n in enumerate([50, 21, 90, 34, 7])})
    steps = trace_mixed(requests, seed=5, live_max=3)
    assert max(len(e) for e, _ in steps) >= 3, "the trace should batch several requests"
    stepper = engines(name, dtype, capacity_tokens=max_live_tokens(steps), max_requests=3)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/mixed")
    assert stepper.cache.pages_reused > 0, "the pool was sized so that pages must be used again"
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_gives_each_request_what_it_gets_alone(engines, dtype):
    """Unequal requests side by side against each alone, in portions that cut windows and pages."""
    from tesseract_b200.engine import StepEntry

    name = "a"
    requests = make_requests(name)
    alone = replay(engines(name, dtype), trace_portions(requests, sizes=(9, 2, 30, 5)))
    together = {}
    stepper = engines(name, dtype)
    at = {rid: 0 for rid in requests}
    for rid in requests:
        assert stepper.cache.admit(rid)
    sizes = [9, 2, 30, 5]
    turn = 0
    while any(at[rid] < len(t) for rid, t in requests.items()):
        batch, meta = [], []
        for rid, tokens in requests.items():
            if at[rid] >= len(tokens):
                continue
            size = sizes[turn % 4]
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
@pytest.mark.parametrize("name", ["a", "d", "e"])
def test_long_decoding_while_the_windows_move(engines, folders, name, dtype):
    tokens = random_tokens(TINY_PEKODRA[name]["vocab"], 180, seed=77)
    requests = {"long": tokens}
    steps = trace_tail(requests, tail=170)          # ten tokens of prompt, then 170 decoded one by one
    stepper = engines(name, dtype, capacity_tokens=192)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/long decode")
    assert stepper.cache.used_pages() == 0


def test_pages_behind_the_window_go_back_while_the_request_lives(engines):
    """Model "d" has windows of 1 and 17 positions and pages of 16: a request of 200 tokens never holds more than a few
    pages a group, far fewer than its thirteen."""
    from tesseract_b200.engine import StepEntry

    stepper = engines("d", "float32", capacity_tokens=96)     # six pages: fewer than the request's 200 tokens take
    assert stepper.cache.admit("one")
    tokens = random_tokens(TINY_PEKODRA["d"]["vocab"], 200, seed=5)
    paged = sum(1 for g in stepper.cache.groups if g.pool is not None)
    assert paged == 2                                           # one group a window
    for at in range(0, 200, 10):
        stepper.step([StepEntry("one", tokens[at:at + 10], [9])])
        assert stepper.cache.used_pages() <= 3 * paged
    stepper.cache.release("one")
    stepper.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["a", "b", "e"])
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
            if got != best and margin > limit and dtype == "bfloat16":
                # what rounding to bfloat16 alone does to this position's logits in the plain model (another expert
                # of two nearly equal ones, for instance) bounds what the engine's token may lose
                coarse = plain.forward(config, tensors, tokens, round_to=torch.bfloat16)[-1].numpy()
                limit = max(limit, 3.0 * float(np.abs(coarse - logits).max()))
            assert got == best or margin <= limit, f"{name}/{dtype}: token {k} is {got}, plain says {best}"
            tokens.append(got)
    assert llm.stepper.cache.used_pages() == 0
    if graphs:      # decode steps and full prompt portions were replayed as graphs, not issued launch by launch
        assert llm.stepper.graphs.safe and llm.stepper.graphs.replays >= steps - 2
        assert llm.stepper.chunk_graphs.replays >= 1
    del llm
    torch.cuda.empty_cache()


def test_replay_program_runs_a_pekodra_folder(folders, tmp_path):
    """``bin/trace_run`` picks the model class by ``config.json`` and writes the logits of the wanted places."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config, tensors = plain.load_folder(folders("c"))
    tokens = random_tokens(config["vocab"], 30, seed=9)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": tokens[20:], "want": [9]}], "end": ["a"]})]
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders("c"), "--dtype",
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
    folder = folders("a")
    common = [sys.executable, os.path.join(root, "bin", "tesseract"), "--model-path", folder, "--kv-capacity-tokens",
              "256", "--max-running", "2", "--dtype", "float32"]
    done = subprocess.run(common + ["--prompt-ids", "5,6,7,8", "--random-prompt", "11", "--max-tokens", "4",
                                    "--temperature", "0", "--ignore-eos", "--json", "--check-weights"],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
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
    assert "kernel plan for Pekodra" in shown.stdout
    assert "mixer 'normed_attention'" in shown.stdout and "feed-forward 'routed_experts'" in shown.stdout


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34])
def test_random_configurations_match_plain_in_float32(tmp_path, seed):
    """Configurations drawn at random (feed-forward kinds, loops, every size and constant), each whole, with a
    decoded tail, in portions and in mixed batches."""
    import random

    from tesseract_b200.engine import load_model, make_stepper
    from tesseract_b200.weights.random_init import write_random_model
    from tests.pekodra_models import random_config

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


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34, 55, 89])
def test_random_configurations_match_plain_in_bfloat16(tmp_path, seed):
    """The same configurations in bfloat16 (products of odd sizes, head sizes on and off the tensor-core kernels), whole,
    with a decoded tail and in mixed batches, the plain model under the engine's choice of experts."""
    import random

    from tesseract_b200.engine import load_model, make_stepper
    from tesseract_b200.weights.random_init import write_random_model
    from tests.pekodra_models import random_config

    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "model"), config, seed=seed)
    r = random.Random(seed + 2000)
    lengths = [1, r.randint(2, 40), r.randint(41, 140), r.randint(260, 330), r.randint(5, 90)]
    requests = {f"q{i}": random_tokens(config["vocab"], n, seed=seed * 10 + i) for i, n in enumerate(lengths)}
    model = load_model(folder, dtype="bfloat16")
    for name, steps in (("whole", trace_whole(requests)), ("tail", trace_tail(requests, tail=20)),
                        ("mixed", trace_mixed(requests, seed=seed, live_max=4))):
        stepper = make_stepper(model, capacity_tokens=max(1024, max_live_tokens(steps)), max_requests=4)
        replay_against_plain(stepper, steps, folder, requests, "bfloat16", f"seed {seed}/{name}", measured_noise=True)
        assert stepper.cache.used_pages() == 0


def test_the_library_and_the_plan_agree_on_the_tensor_core_head_sizes():
    from tesseract_b200 import kernels
    from tesseract_b200.csrc.build import load_library

    lib = load_library("attention_prompt_mma")
    for d in (8, 16, 48, 64, 96, 128, 256):
        for dv in (8, 48, 64, 96, 128, 256):
            assert bool(lib.tb_attention_prompt_mma_supported(d, dv)) == kernels.attention_prompt_mma_supported(torch.bfloat16, d, dv)
    assert not kernels.attention_prompt_mma_supported(torch.float32, 64, 64)
