"""Doderax on the GPU against the plain implementation (tests/plain_doderax.py): every mechanism's kernel alone, then
whole models through the engine's step function, cache manager and scheduler: prompts whole, token by token, in
portions down to two tokens, in batches of unequal requests, with pages and state slots that change hands, with
windows and kept first tokens at page borders, in long decoding, and greedy generation through the entry point."""

import json
import math

import numpy as np
import pytest
import torch

import plain_doderax as plain
from doderax_configs import ALL, PAGE_SIZES, make_folder, random_config
from helpers import TOL, Trace, random_ids, run_trace

pytestmark = pytest.mark.gpu
F64 = torch.float64


def device():
    return torch.device("cuda", 0)


def close(got, want, tol, what=""):
    got = got.detach().double().cpu() if isinstance(got, torch.Tensor) else torch.as_tensor(got, dtype=F64)
    want = want.detach().double().cpu() if isinstance(want, torch.Tensor) else torch.as_tensor(want, dtype=F64)
    error = (got - want).abs().max().item()
    bound = tol * max(1.0, want.abs().max().item())
    assert math.isfinite(error) and error <= bound, f"{what}: max |diff| {error:.3e} > {bound:.3e}"


def close_logits(got, want, dtype, what=""):
    """Logits [positions, vocab] of a whole model.  float32: every value within the tolerance.  bfloat16: the
    projections are rounded to 8 bits of mantissa, and where a recurrent head reads almost nothing out of its state
    (a query nearly orthogonal to the few keys written so far, at a request's first tokens) the per-head norm that
    follows magnifies that rounding to several per cent of the logits at that one position; so positions are judged
    by their relative root-mean-square error: nine in ten within the tolerance, none beyond five times it.  A lost
    state, a tap from the wrong token or a window one token off is an error of order one at most positions."""
    if dtype == "float32":
        return close(got, want, TOL[dtype], what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
    assert np.isfinite(relative).all(), f"{what}: not finite"
    assert np.quantile(relative, 0.9) <= TOL[dtype] and relative.max() <= 5 * TOL[dtype], \
        f"{what}: relative error of positions: 90% {np.quantile(relative, 0.9):.3e}, max {relative.max():.3e}"


def batch_description(portions, slots):
    """Device tensors describing packed rows: portions = tokens per request row."""
    starts = np.concatenate([[0], np.cumsum(portions)]).astype(np.int32)
    row_of_token = np.repeat(np.arange(len(portions)), portions).astype(np.int32)
    to = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=device())
    return to(row_of_token), to(starts), to(slots), to(np.zeros(int(starts[-1])))


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_hashes_a_token_with_the_one_before(dtype):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(0)
    vocab, hidden, buckets = 50, 24, 13
    table = torch.randn(vocab, hidden, generator=generator).to(dtype).to(device())
    pairs = torch.randn(buckets + 1, hidden, generator=generator).to(dtype).to(device())
    ids = torch.tensor([3, 49, 0, 7, 7, 21], dtype=torch.int32, device=device())
    before = torch.tensor([-1, 3, 49, -1, 7, 7], dtype=torch.int32, device=device())
    out = torch.empty(6, hidden, dtype=torch.float32, device=device())
    kernels.embed_pairs(table, pairs, ids, before, out, 1000003, 77, 1.0)
    rows = [buckets if b < 0 else (b * 1000003 + i * 77) % buckets for b, i in zip(before.tolist(), ids.tolist())]
    want = table.double()[ids.long()] + pairs.double()[torch.tensor(rows, device=device())]
    close(out, want, 1e-6, "embed_pairs")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_gelu_and_the_sum_of_normed_branches(dtype, tol):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(1)
    x = (torch.randn(37, 50, generator=generator) * 3).to(dtype).to(device())
    want = plain.gelu_tanh(x.double().cpu())
    kernels.gelu_tanh(x)
    close(x, want, tol, "gelu_tanh")
    hidden = 88
    branches = [torch.randn(9, hidden, generator=generator, dtype=torch.float32).to(device()) * (b + 1) for b in range(3)]
    weights = [torch.randn(hidden, generator=generator, dtype=torch.float32).to(device()) for _ in range(3)]
    residual = torch.randn(9, hidden, generator=generator, dtype=torch.float32).to(device())
    want = residual.double().cpu() + 0.25 * sum(plain.unit_rms(b.double().cpu(), 1e-3) * w.double().cpu()
                                                for b, w in zip(branches, weights))
    kernels.add_normed_branches(branches, weights, residual, 1e-3, 0.25)
    close(residual, want, 2e-6, "add_normed_branches")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_short_convolution_carries_its_last_inputs_between_portions(dtype, taps):
    """Two requests fed in portions of 1, 2, 3 and more tokens, interleaved in one batch, in state slots 2 and 0."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(taps)
    channels, width = 70, 96                                    # the convolved columns are a range of wider rows
    lengths = [23, 17]
    inputs = [torch.randn(n, channels, generator=generator).to(dtype) for n in lengths]
    weight = (torch.randn(channels, taps, generator=generator) * 0.7).to(dtype)
    want = [plain.short_conv_silu(x.double(), weight.double()) for x in inputs]
    tail = torch.full((3, max(taps - 1, 0), channels), 0.0, dtype=torch.float32, device=device())
    got = [[], []]
    cursors = [0, 0]
    for portions in ([1, 2], [2, 1], [3, 1], [1, 5], [9, 2], [7, 6]):
        rows = torch.zeros(sum(portions), width, dtype=dtype)
        at = 0
        for r, count in enumerate(portions):
            rows[at:at + count, 8:8 + channels] = inputs[r][cursors[r]:cursors[r] + count]
            at += count
        rows = rows.to(device())
        row_of_token, starts, slots, positions = batch_description(portions, [2, 0])
        out = torch.empty(sum(portions), channels, dtype=torch.float32, device=device())
        kernels.short_conv_silu(rows[:, 8:8 + channels], weight.to(device()), tail, row_of_token, starts, slots,
                                positions, out)
        at = 0
        for r, count in enumerate(portions):
            got[r].append(out[at:at + count].cpu())
            cursors[r] += count
            at += count
    for r in range(2):
        close(torch.cat(got[r]), want[r], 2e-6, f"short_conv_silu, request {r}, {taps} taps")
    assert torch.all(tail[1] == 0), "the state of a slot nobody used was written"


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("heads,kv_heads,key_dim,value_dim,taps", [(2, 2, 64, 32, 4), (6, 2, 24, 40, 1), (1, 1, 200, 3, 2),
                                                                     (4, 1, 96, 128, 3), (3, 3, 8, 1, 1), (2, 1, 30, 5, 4),
                                                                     (2, 2, 128, 9, 2), (1, 1, 1, 4, 3)])
def test_delta_rule_against_the_plain_recurrence(per_channel, heads, kv_heads, key_dim, value_dim, taps):
    """The parallel pass (convolution, unit vectors, gates) and the recurrence: whole sequences, and the same cut into
    portions with state and convolution tail carried; two requests in one batch beside a slot of somebody else."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(heads * 100 + key_dim)
    lengths = [40, 29]
    width = 2 * kv_heads * key_dim + heads * value_dim
    decay_width = heads * key_dim if per_channel else heads
    a_log = torch.rand(heads, generator=generator) * 2 - 1.5
    dt_bias = torch.randn(decay_width, generator=generator)
    conv = torch.randn(width, taps, generator=generator) * 0.8
    data, want = [], []
    for n in lengths:
        x = torch.randn(n, width, generator=generator)
        beta_raw = torch.randn(n, heads, generator=generator) * 2
        decay_raw = torch.randn(n, decay_width, generator=generator) * 2
        data.append((x, beta_raw, decay_raw))
        mixed = plain.short_conv_silu(x.double(), conv.double())
        q = mixed[:, :kv_heads * key_dim].reshape(n, kv_heads, key_dim)
        k = mixed[:, kv_heads * key_dim:2 * kv_heads * key_dim].reshape(n, kv_heads, key_dim)
        v = mixed[:, 2 * kv_heads * key_dim:].reshape(n, heads, value_dim)
        raw = (decay_raw.double() + dt_bias.double())
        decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * plain.softplus(raw).reshape(n, heads, -1))
        decay = decay.expand(n, heads, key_dim)
        want.append(plain.delta_rule(q, k, v, torch.sigmoid(beta_raw.double()), decay).reshape(n, heads * value_dim))
    for cuts in ([lengths], [[1, 1], [2, 1], [5, 2], [1, 7], [31, 18]]):
        state = torch.zeros(4, heads, value_dim, key_dim, dtype=torch.float32, device=device())
        tail = torch.zeros(4, taps - 1, width, dtype=torch.float32, device=device())
        state[2] = 7.0                                           # a slot of somebody else
        got, cursors = [[], []], [0, 0]
        for portions in cuts:
            pieces = [[d[r][cursors[r]:cursors[r] + portions[r]] for r in range(2)] for d in zip(*data)]
            x, beta_raw, decay_raw = (torch.cat(piece).contiguous().to(device()) for piece in pieces)
            row_of_token, starts, slots, positions = batch_description(portions, [3, 1])
            tokens = sum(portions)
            prepared = torch.empty(tokens, width, dtype=torch.float32, device=device())
            beta = torch.empty(tokens, heads, dtype=torch.float32, device=device())
            decay = torch.empty(tokens, decay_width, dtype=torch.float32, device=device())
            kernels.delta_rule_prepare(x, conv.to(device()), tail, beta_raw, decay_raw, dt_bias.to(device()),
                                       a_log.to(device()), row_of_token, starts, slots, positions, prepared, beta, decay,
                                       heads, kv_heads, key_dim, value_dim)
            out = torch.empty(tokens, heads * value_dim, dtype=torch.float32, device=device())
            kernels.delta_rule_scan(prepared, beta, decay, state, starts, slots, positions, out, heads, kv_heads,
                                    key_dim, value_dim)
            at = 0
            for r, count in enumerate(portions):
                got[r].append(out[at:at + count].cpu())
                cursors[r] += count
                at += count
        for r in range(2):
            close(torch.cat(got[r]), want[r], 2e-5, f"delta rule, request {r}, cuts {len(cuts)}")
        assert torch.all(state[2] == 7.0) and torch.all(state[0] == 0.0) and torch.all(tail[0] == 0.0)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("sigmoid_gate", [False, True])
def test_gated_head_norm(dtype, tol, sigmoid_gate):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(5)
    tokens, heads, value_dim = 11, 3, 40
    read = torch.randn(tokens, heads * value_dim, generator=generator) * 0.01       # small: eps matters
    packed = torch.randn(tokens, 8 + heads * value_dim, generator=generator).to(dtype)
    weight = torch.randn(value_dim, generator=generator)
    out = torch.empty(tokens, heads * value_dim, dtype=dtype, device=device())
    kernels.gated_head_norm(read.to(device()), packed.to(device())[:, 8:], weight.to(device()), out, heads, value_dim,
                            1e-5, sigmoid_gate)
    gate = packed[:, 8:].double().reshape(tokens, heads, value_dim)
    act = torch.sigmoid(gate) if sigmoid_gate else plain.silu(gate)
    want = plain.unit_rms(read.double().reshape(tokens, heads, value_dim), 1e-5) * weight.double() * act
    close(out, want.reshape(tokens, -1), tol, "gated_head_norm")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("page_size,window,keep_first", [(8, 9, 20), (16, 16, 16), (4, 30, 1), (8, 5, 0), (8, 100, 3)])
def test_attention_window_with_kept_first_tokens_one_key_stands_out(dtype, tol, page_size, window, keep_first):
    """Queries at several positions, each made to look at exactly one key: the last one inside its window, the first
    one outside it, the last kept token, the first one that is not kept, keys at page borders.  The standing-out key's
    value is unlike every other, so seeing a key that should be hidden, or missing one, changes the result by order 1.
    Pages are shuffled; values are 12 wide where keys are 16."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(window * 10 + keep_first)
    length, heads, kv_heads, head_dim, value_dim = 90, 4, 2, 16, 12
    keys = torch.randn(length, kv_heads, head_dim, generator=generator) * 0.1
    values = torch.randn(length, kv_heads, value_dim, generator=generator)
    pages = -(-length // page_size)
    order = torch.randperm(pages + 3, generator=generator)[:pages]
    k_pages = torch.full(((pages + 3) * page_size, kv_heads, head_dim), 50.0)
    v_pages = torch.full(((pages + 3) * page_size, kv_heads, value_dim), -50.0)
    for position in range(length):
        slot = int(order[position // page_size]) * page_size + position % page_size
        k_pages[slot], v_pages[slot] = keys[position], values[position]
    cases = []
    for position in (length - 1, 57, window + keep_first + 2, keep_first, 0, page_size, page_size - 1):
        position = min(max(position, 0), length - 1)
        for target in (position - window + 1, position - window, keep_first - 1, keep_first, position,
                       (position // page_size) * page_size, (position // page_size) * page_size - 1):
            if 0 <= target <= position:
                cases.append((position, target))
    queries = torch.zeros(len(cases), heads * head_dim)
    for row, (position, target) in enumerate(cases):
        for head in range(heads):
            queries[row, head * head_dim:(head + 1) * head_dim] = keys[target, head // (heads // kv_heads)] * 400.0
    table = order.to(torch.int32)[None, :].repeat(len(cases), 1).contiguous()
    positions = torch.tensor([p for p, _ in cases], dtype=torch.int32)
    out = torch.empty(len(cases), heads * value_dim, dtype=dtype, device=device())
    rows = torch.arange(len(cases), dtype=torch.int32)
    kernels.paged_attention_generic(queries.to(dtype).to(device()), out, k_pages.to(dtype).to(device()),
                                    v_pages.to(dtype).to(device()), table.to(device()), rows.to(device()),
                                    positions.to(device()), page_size, heads, kv_heads, head_dim, 1.0, window,
                                    value_dim=value_dim, keep_first=keep_first)
    k64, v64 = keys.to(dtype).double(), values.to(dtype).double()
    for row, (position, target) in enumerate(cases):
        q = queries[row].to(dtype).double().reshape(heads, head_dim)
        mask = plain.visible(position + 1, window, keep_first)[position]
        for head in range(heads):
            scores = (k64[:position + 1, head // 2] @ q[head]).masked_fill(~mask, -math.inf)
            want = torch.softmax(scores, dim=-1) @ v64[:position + 1, head // 2]
            close(out[row, head * value_dim:(head + 1) * value_dim], want, tol,
                  f"query {position} looking at key {target} (window {window}, kept {keep_first}, page {page_size})")


@pytest.mark.parametrize("head_dim,tcgen05", [(64, False), (128, False), (128, True)])
@pytest.mark.parametrize("page_size,window,keep_first", [(16, 70, 5), (8, 40, 66), (16, 64, 64), (32, 100, 130), (16, 30, 1),
                                                         (16, 128, 128), (16, 200, 129)])
def test_tile_attention_with_kept_first_keys(head_dim, tcgen05, page_size, window, keep_first):
    """The tensor-core tile kernels (bfloat16: mma.sync, and tcgen05 where the head is 128 wide) on a portion of 150 queries after 150 cached keys, beside a single
    decoded token of another request: every query is made to look at one key at an edge (the last one inside its
    window, the first one outside, the last kept key, the first one not kept)."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(window + keep_first)
    heads, kv_heads = 4, 2
    lengths, portions = [300, 211], [150, 1]
    dtype = torch.bfloat16
    pages_each = [-(-n // page_size) for n in lengths]
    order = torch.randperm(sum(pages_each) + 4, generator=generator)
    k_pages = torch.full(((sum(pages_each) + 4) * page_size, kv_heads, head_dim), 30.0)
    v_pages = torch.full(((sum(pages_each) + 4) * page_size, kv_heads, head_dim), -30.0)
    table = torch.full((2, max(pages_each)), -1, dtype=torch.int32)
    keys, values, queries, want = [], [], [], []
    at = 0
    for r, n in enumerate(lengths):
        table[r, :pages_each[r]] = order[at:at + pages_each[r]].to(torch.int32)
        at += pages_each[r]
        k = (torch.randn(n, kv_heads, head_dim, generator=generator) * 0.1).to(dtype)
        v = torch.randn(n, kv_heads, head_dim, generator=generator).to(dtype)
        for position in range(n):
            slot = int(table[r, position // page_size]) * page_size + position % page_size
            k_pages[slot], v_pages[slot] = k[position].float(), v[position].float()
        q = torch.zeros(portions[r], heads, head_dim)
        for local in range(portions[r]):
            position = n - portions[r] + local
            choices = [t for t in (position - window + 1, position - window, keep_first - 1, keep_first, position)
                       if 0 <= t <= position]
            target = choices[int(torch.randint(len(choices), (1,), generator=generator))]
            for head in range(heads):
                q[local, head] = k[target, head // 2].float() * (600.0 / (head_dim / 16))
        q = q.to(dtype)
        mask = plain.visible(n, window, keep_first)[n - portions[r]:]
        for head in range(heads):
            scores = (q[:, head].double() @ k[:, head // 2].double().T).masked_fill(~mask, -math.inf)
            want.append((r, head, torch.softmax(scores, dim=-1) @ v[:, head // 2].double()))
        queries.append(q.reshape(portions[r], heads * head_dim))
    # packed rows: the single token first, as the engine packs them
    packed = torch.cat([queries[1], queries[0]]).to(device())
    starts = torch.tensor([0, 1, 151], dtype=torch.int32, device=device())
    contexts = torch.tensor([lengths[1], lengths[0]], dtype=torch.int32, device=device())
    tables = torch.stack([table[1], table[0]]).contiguous().to(device())
    out = torch.empty(151, heads * head_dim, dtype=dtype, device=device())
    kernels.prefill_attention(packed, out, k_pages.to(dtype).to(device()), v_pages.to(dtype).to(device()), tables, starts,
                              contexts, page_size, heads, kv_heads, head_dim, 1.0, window, tensor_cores=tcgen05,
                              keep_first=keep_first)
    assert kernels.prefill_attention_error() == 0
    for r, head, expected in want:
        rows = out[1:151] if r == 0 else out[0:1]
        close(rows[:, head * head_dim:(head + 1) * head_dim], expected, 2e-2,
              f"request {r} head {head} (window {window}, kept {keep_first}, page {page_size})")


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("page_size,window,keep_first", [(16, 70, 5), (8, 40, 66), (16, 256, 16), (32, 100, 130), (16, 30, 1),
                                                         (16, 600, 7)])
def test_split_key_decode_attention_with_kept_first_keys(head_dim, page_size, window, keep_first):
    """Single decoded tokens of requests that hold 1 to 1,000 keys, split over partitions of 256 keys (bfloat16,
    mma.sync): each query looks at one key at an edge of its window or of the kept keys."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(window * 7 + keep_first)
    heads, kv_heads = 6, 2
    lengths = [1000, 300, window + keep_first + 1, keep_first, 1, 71, 513]
    lengths = [max(1, n) for n in lengths]
    dtype = torch.bfloat16
    pages_each = [-(-n // page_size) for n in lengths]
    order = torch.randperm(sum(pages_each) + 4, generator=generator)
    k_pages = torch.full(((sum(pages_each) + 4) * page_size, kv_heads, head_dim), 30.0)
    v_pages = torch.full(((sum(pages_each) + 4) * page_size, kv_heads, head_dim), -30.0)
    table = torch.full((len(lengths), max(pages_each)), -1, dtype=torch.int32)
    queries, want, at = [], [], 0
    for r, n in enumerate(lengths):
        table[r, :pages_each[r]] = order[at:at + pages_each[r]].to(torch.int32)
        at += pages_each[r]
        k = (torch.randn(n, kv_heads, head_dim, generator=generator) * 0.1).to(dtype)
        v = torch.randn(n, kv_heads, head_dim, generator=generator).to(dtype)
        for position in range(n):
            slot = int(table[r, position // page_size]) * page_size + position % page_size
            k_pages[slot], v_pages[slot] = k[position].float(), v[position].float()
        position = n - 1
        choices = [t for t in (position - window + 1, position - window, keep_first - 1, keep_first, position)
                   if 0 <= t <= position]
        q = torch.zeros(heads, head_dim)
        for head in range(heads):
            target = choices[(r + head) % len(choices)]
            q[head] = k[target, head // 3].float() * (600.0 / (head_dim / 16))
        q = q.to(dtype)
        mask = plain.visible(n, window, keep_first)[position]
        rows = []
        for head in range(heads):
            scores = (k[:, head // 3].double() @ q[head].double()).masked_fill(~mask, -math.inf)
            rows.append(torch.softmax(scores, dim=-1) @ v[:, head // 3].double())
        want.append(torch.cat(rows))
        queries.append(q.reshape(heads * head_dim))
    rows = len(lengths)
    packed = torch.stack(queries).to(device())
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=device())
    out = torch.empty(rows, heads * head_dim, dtype=dtype, device=device())
    partition, count, floats = kernels.decode_attention_kept_plan(rows, heads, head_dim, max(lengths))
    assert count > 1
    scratch = torch.empty(floats, dtype=torch.float32, device=device())
    numbering = torch.empty(rows, dtype=torch.int32, device=device())
    kernels.decode_attention(packed, out, k_pages.to(dtype).to(device()), v_pages.to(dtype).to(device()),
                             table.contiguous().to(device()), positions, page_size, heads, kv_heads, head_dim, 1.0, window,
                             partition, count, scratch, keep_first=keep_first, numbering=numbering)
    for r in range(rows):
        close(out[r], want[r], 2e-2, f"request of {lengths[r]} keys (window {window}, kept {keep_first}, page {page_size})")


# ------------------------------------------------------------------------------ whole models through the engine
def load(folder, dtype, page_size, pages, requests=4, graphs=False):
    from libmir_b200 import CacheConfig, CudaConfig, Library, RuntimeConfig, SchedulerConfig
    runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=page_size, block_count=pages),
                            scheduler=SchedulerConfig(max_batch_requests=requests),
                            cuda=CudaConfig(decode_graphs=graphs), dtype=dtype)
    return Library(runtime).load(folder)


def reference(folder, ids):
    config, weights = plain.read_model(folder)
    return plain.forward(config, weights, list(ids)).numpy()


def feed(model, name, ids, cuts):
    """Feed `ids` in portions of the given sizes (the last repeated), wanting every position; returns logits [n, V]."""
    from libmir_b200 import StepEntry
    model.admit(name)
    out, cursor, turn = [], 0, 0
    while cursor < len(ids):
        size = min(cuts[min(turn, len(cuts) - 1)], len(ids) - cursor)
        result = model.step([StepEntry(name, ids[cursor:cursor + size], range(size))])
        out.append(result.logits.cpu().numpy().copy())
        cursor += size
        turn += 1
    model.release(name)
    return np.concatenate(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole_prompts_token_by_token_and_portions(tmp_path, name, dtype):
    """A prompt whole; the same token by token from its first token (150 single steps: long decoding, windows that
    pass many times, the first tokens of a sequence); and in portions of changing size down to two tokens."""
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=3, dtype=dtype)
    rng = np.random.default_rng(7)
    ids = random_ids(rng, config["vocab"], 150)
    want = reference(folder, ids)
    model = load(folder, dtype, PAGE_SIZES[name], 40)
    whole = feed(model, "whole", ids, [len(ids)])
    close_logits(whole, want, dtype, f"{name}/{dtype} whole")
    single = feed(model, "single", ids, [1])
    close_logits(single, want, dtype, f"{name}/{dtype} token by token")
    portions = feed(model, "portions", ids, [2, 3, 1, 7, 2, 16, 5, 2, 33, 1, 2, 9])
    close_logits(portions, want, dtype, f"{name}/{dtype} portions")
    late = feed(model, "late", ids, [118, 1])                      # most of it whole, the last 32 one by one
    close_logits(late, want, dtype, f"{name}/{dtype} prompt then decoding")
    if dtype == "float32":
        # 32-bit results do not depend on the cut at all: the recurrence walks a request's tokens in order, attention
        # reduces a query's keys in an order that depends on its position alone, products reduce in ascending order
        assert np.array_equal(whole, single) and np.array_equal(whole, portions) and np.array_equal(whole, late)
    for group in model.cache_stats()["groups"]:
        assert group["free"] == group["pages"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["V", "W", "X", "Z"])
def test_batches_of_unequal_requests_with_pages_and_slots_that_change_hands(tmp_path, name, dtype):
    """Up to three live requests of unequal lengths, portions of some beside single tokens of others, requests that
    sit a step out, in a pool so small that pages and state slots are used again; every request against itself
    alone (the plain implementation)."""
    from libmir_b200 import StepEntry
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=5, dtype=dtype)
    rng = np.random.default_rng(11)
    lengths = [70, 31, 96, 18, 55, 40, 77]
    requests = [random_ids(rng, config["vocab"], n) for n in lengths]
    want = [reference(folder, ids) for ids in requests]
    page = PAGE_SIZES[name]
    model = load(folder, dtype, page, 3 * (-(-96 // page)) + 2, requests=3)
    queue, live, got = list(range(len(requests))), {}, {i: [] for i in range(len(requests))}
    while queue or live:
        while queue and len(live) < 3:
            index = queue.pop(0)
            model.admit(f"r{index}")
            live[index] = 0
        entries, ended = [], []
        for index in list(live):
            cursor, ids = live[index], requests[index]
            if len(live) > 1 and rng.random() < 0.25:
                continue
            decode_from = max(2, len(ids) - 20)
            size = 1 if cursor >= decode_from else min(int(rng.integers(2, 19)), decode_from - cursor)
            entries.append(StepEntry(f"r{index}", ids[cursor:cursor + size], range(size)))
            live[index] = cursor + size
            if live[index] == len(ids):
                ended.append(index)
        if not entries:
            continue
        result = model.step(entries)
        logits, at = result.logits.cpu().numpy(), 0
        for entry in entries:
            got[int(entry.request_id[1:])].append(logits[at:at + len(entry.tokens)].copy())
            at += len(entry.tokens)
        for index in ended:
            model.release(f"r{index}")
            del live[index]
        model.cache.check()
    for index in range(len(requests)):
        close_logits(np.concatenate(got[index]), want[index], dtype, f"{name}/{dtype} request {index} in a mixed batch")
    stats = model.cache_stats()
    assert stats["free_slots"] == 3
    for group in stats["groups"]:
        assert group["free"] == group["pages"] and group["reused"] > 0
    assert stats["groups"] or name == "V"


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_greedy_generation_through_the_scheduler(tmp_path, name, graphs):
    """Model.generate_batch (scheduler, sampler, decode steps as captured graphs or not) against the plain
    implementation choosing greedily; float32, so that equal choices are expected wherever the best two logits are
    not closer than the tolerance."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=9, dtype="float32")
    plain_config, weights = plain.read_model(folder)
    rng = np.random.default_rng(2)
    prompts = [random_ids(rng, config["vocab"], n) for n in (5, 23, 1)]
    model = load(folder, "float32", PAGE_SIZES[name], 48, graphs=graphs)
    outputs = model.generate_batch([GenerationRequest(p, GenerationOverrides(max_tokens=12, ignore_eos=True))
                                    for p in prompts])
    for prompt, output in zip(prompts, outputs):
        assert len(output.token_ids) == 12
        ids = list(prompt)
        for token in output.token_ids:
            logits = plain.forward(plain_config, weights, ids)[-1]
            best = int(torch.argmax(logits))
            assert token == best or float(logits[best] - logits[token]) < 1e-4, \
                f"{name}: the engine chose {token}, the plain implementation {best}"
            ids.append(token)
    if graphs:
        assert model.runner._graphs is not None and len(model.runner._graphs.graphs) > 0


def test_trace_runner_picks_the_design_by_its_configuration(tmp_path):
    """bin/trace_run as a user runs it: the model class comes from config.json; prompts in portions, decoded tokens,
    a pool that holds less than all requests together."""
    config = ALL["Z"]
    folder = make_folder(tmp_path / "model", config, seed=4, dtype="bfloat16")
    (folder / "config.json").write_text(json.dumps(dict(config, vocab_size=config["vocab"])))   # (helpers read this key)
    rng = np.random.default_rng(3)
    requests = {f"q{i}": random_ids(rng, config["vocab"], n) for i, n in enumerate((100, 64, 37))}
    want = {name: reference(folder, ids) for name, ids in requests.items()}
    for dtype in ("bfloat16", "float32"):
        trace = Trace()
        for name, ids in requests.items():
            trace.step([(name, ids[:len(ids) - 10], [0, len(ids) - 11])])
            for position in range(len(ids) - 10, len(ids)):
                trace.step([(name, ids[position:position + 1], [0])], end=[name] if position == len(ids) - 1 else [])
        results = run_trace(folder, dtype, trace, tmp_path / f"out-{dtype}", max_tokens=128,
                            extra_args=["--page-size", "8"])
        for index, rows in enumerate(trace.expect):
            for row, (name, position) in enumerate(rows):
                close(results[index][row], want[name][position], TOL[dtype], f"trace {dtype} {name}@{position}")


@pytest.mark.parametrize("rows", [1, 8, 32, 33, 127, 128, 300])
def test_up_projection_with_the_activation_in_its_epilogue(rows):
    """gelu_tanh(x W^T) in bfloat16 through every product the row count selects (weight streaming, the library with
    the activation kernel, the many-rows tcgen05 kernel) against float64."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(rows)
    k, n = 96, 200
    x = torch.randn(rows, k, generator=generator).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=generator) * 0.3).to(torch.bfloat16)
    out = torch.empty(rows, n, dtype=torch.bfloat16, device=device())
    alloc = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=device())
    kernels.linear_gelu(x.to(device()), w.to(device()), out, alloc=alloc)
    close(out, plain.gelu_tanh(x.double() @ w.double().T), 1e-2, f"linear_gelu, {rows} rows")
    assert kernels.stream_linear_error() == 0 and kernels.tensor_core_linear_error() == 0


def test_generate_command_line(tmp_path):
    """bin/generate on a model folder of the design: two prompts as one batch, greedy, against the plain
    implementation; and one prompt sampled with a seed, twice, for the same tokens."""
    import subprocess
    import sys
    from helpers import ROOT
    config = ALL["X"]
    folder = make_folder(tmp_path / "model", config, seed=12, dtype="float32")
    plain_config, weights = plain.read_model(folder)
    command = [sys.executable, str(ROOT / "bin" / "generate"), str(folder), "--dtype", "float32", "--block-size", "8",
               "--block-count", "64", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(command + ["--prompt-ids", "5,9,200,33;7", "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    outputs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(outputs) == 2
    for prompt, output in zip(([5, 9, 200, 33], [7]), outputs):
        ids = list(prompt)
        for token in output["token_ids"]:
            logits = plain.forward(plain_config, weights, ids)[-1]
            best = int(torch.argmax(logits))
            assert token == best or float(logits[best] - logits[token]) < 1e-4
            ids.append(token)
    sampled = [subprocess.run(command + ["--prompt-ids", "1,2,3", "--temperature", "0.9", "--top-k", "20", "--seed", "4"],
                              capture_output=True, text=True, timeout=600).stdout for _ in range(2)]
    assert sampled[0] == sampled[1] and "finish_reason=" in sampled[0]


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes nobody chose: a prompt whole, token by token, in portions and as a prompt followed by decoding, in both
    dtypes, against the plain implementation (32-bit: every position within 2e-4 of its logits' root mean square and
    the same bits under every cut; bfloat16: nine positions in ten within the tolerance)."""
    rng = np.random.default_rng(500 + seed)
    config = random_config(rng)
    page = int(rng.choice([4, 8, 16]))
    ids = random_ids(rng, config["vocab"], 100)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=seed, dtype=dtype)
        want = reference(folder, ids)
        model = load(folder, dtype, page, 80)
        outputs = [feed(model, "whole", ids, [len(ids)]), feed(model, "single", ids, [1]),
                   feed(model, "portions", ids, [2, 5, 1, 33, 3, 16, 2, 7]), feed(model, "late", ids, [80, 1])]
        for got in outputs:
            relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
            assert np.isfinite(relative).all(), json.dumps(config)
            if dtype == "float32":
                assert relative.max() <= 2e-4, f"{relative.max():.3e} at {int(relative.argmax())}: {json.dumps(config)}"
            else:
                assert np.quantile(relative, 0.9) <= TOL[dtype], f"{np.quantile(relative, 0.9):.3e}: {json.dumps(config)}"
        if dtype == "float32":
            assert all(np.array_equal(outputs[0], other) for other in outputs[1:]), json.dumps(config)
        model.unload()
