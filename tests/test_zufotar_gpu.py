"""Zufotar on the GPU against the plain implementation (tests/plain_zufotar.py): every mechanism's kernel alone, then
whole models through the engine's step function, cache manager and scheduler: prompts whole, token by token, in
portions down to two tokens, in batches of unequal requests, with pages and state slots that change hands, with keys
far away and at page borders, in long decoding, and greedy generation through the entry point."""

import json
import math

import numpy as np
import pytest
import torch

import plain_zufotar as plain
from helpers import TOL, Trace, random_ids, run_trace
from zufotar_configs import ALL, PAGE_SIZES, make_folder, random_config

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
    """Logits [positions, vocab] of a whole model.  float32: every value within the tolerance.  bfloat16: positions
    are judged by their relative root-mean-square error, nine in ten within the tolerance and all but three in a
    hundred within five times it: where two experts' scores lie closer together than the rounding of the router's
    input, the engine and the 64-bit implementation may choose differently at that one token, and where a recurrent
    head reads almost nothing out of a young state the per-head norm magnifies the projections' rounding.  A lost
    state, a blend with the wrong token, a missed key or a dropped pass is an error of order one at most positions."""
    if dtype == "float32":
        return close(got, want, TOL[dtype], what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
    assert np.isfinite(relative).all(), f"{what}: not finite"
    assert np.quantile(relative, 0.9) <= TOL[dtype] and (relative <= 5 * TOL[dtype]).mean() >= 0.97, \
        f"{what}: relative error of positions: 90% {np.quantile(relative, 0.9):.3e}, max {relative.max():.3e}"


def on_device(tensor, dtype=None):
    return tensor.to(device=device(), dtype=dtype or tensor.dtype).contiguous()


def batch_description(portions, slots, starts_at=None):
    """Device tensors describing packed rows: portions = tokens per request row; positions count from starts_at."""
    starts = np.concatenate([[0], np.cumsum(portions)]).astype(np.int32)
    row_of_token = np.repeat(np.arange(len(portions)), portions).astype(np.int32)
    first = starts_at or [0] * len(portions)
    positions = np.concatenate([np.arange(f, f + n) for f, n in zip(first, portions)]) if len(portions) else []
    to = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=device())
    return to(row_of_token), to(starts), to(slots), to(positions)


DTYPES = [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)]


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_small_elementwise_kernels(dtype, tol):
    """The exact GELU, tanh, the cap on the logits, what a pass of a loop adds, and two norms of the same rows."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(1)
    x = (torch.randn(37, 52, generator=generator) * 2.0).to(dtype)
    for launcher, function in ((kernels.gelu_erf, plain.gelu_erf), (kernels.tanh, torch.tanh)):
        y = on_device(x.clone())
        launcher(y)
        close(y, function(x.double()), tol, launcher.__name__)
    logits = torch.randn(5, 301, generator=generator) * 20.0
    capped = on_device(logits.clone())
    kernels.softcap(capped, 7.5)
    close(capped, 7.5 * torch.tanh(logits.double() / 7.5), 2e-6, "softcap")
    residual, rows, vector = torch.randn(9, 52, generator=generator), torch.randn(9, 52, generator=generator), torch.randn(52, generator=generator)
    for use_rows, use_vector in ((True, True), (False, True), (True, False)):
        r = on_device(residual.clone())
        kernels.add_rows(r, on_device(rows) if use_rows else None, on_device(vector) if use_vector else None)
        close(r, residual + (rows if use_rows else 0) + (vector if use_vector else 0), 1e-6, "add_rows")
    w_a, w_b = 1.0 + torch.randn(52, generator=generator) * 0.3, torch.randn(52, generator=generator)
    out_a, out_b = torch.empty(9, 52, dtype=dtype, device=device()), torch.empty(9, 52, dtype=dtype, device=device())
    kernels.rms_norm_pair(on_device(residual), on_device(w_a), on_device(w_b), 1e-5, out_a, out_b)
    normed = plain.unit_rms(residual.double(), 1e-5)
    close(out_a, normed * w_a, tol, "rms_norm_pair, first")
    close(out_b, normed * w_b, tol, "rms_norm_pair, second")


@pytest.mark.parametrize("rows", [1, 8, 32, 33, 127, 128, 300])
def test_up_projection_with_the_exact_gelu_in_its_epilogue(rows):
    """gelu_erf(x W^T) in bfloat16 through every product the row count selects (weight streaming, the library with
    the activation kernel, the many-rows tcgen05 kernel) against float64; and in float32."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(rows)
    k, n = 96, 200
    x = torch.randn(rows, k, generator=generator).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=generator) * 0.3).to(torch.bfloat16)
    alloc = lambda shape, dtype: torch.empty(shape, dtype=dtype, device=device())
    want = plain.gelu_erf(x.double() @ w.double().T)
    out = torch.empty(rows, n, dtype=torch.bfloat16, device=device())
    kernels.linear_gelu(on_device(x), on_device(w), out, alloc=alloc, exact=True)
    close(out, want, 1e-2, f"linear_gelu exact, {rows} rows")
    out32 = torch.empty(rows, n, device=device())
    kernels.linear_gelu(on_device(x.float()), on_device(w.float()), out32, alloc=alloc, exact=True)
    close(out32, want, 1e-5, f"linear_gelu exact in 32-bit, {rows} rows")
    assert kernels.stream_linear_error() == 0 and kernels.tensor_core_linear_error() == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("interleaved", [True, False])
def test_rotation_of_strided_rows(dtype, tol, interleaved):
    """rope_rows on a strided view, into another buffer and in place; positions up to thousands, a magnitude."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(2)
    tokens, heads, width, rotary = 11, 3, 20, 12
    rot = {"dims": rotary, "base": 1000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}
    freq, magnitude = plain.rotary_table(rot)
    x = torch.randn(tokens, heads, width, generator=generator).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 63, 64, 65, 1000, 4095, 4096, 7], dtype=torch.int32)
    part = x[:, :, 4:4 + rotary].double()
    if interleaved:
        want = plain.rotate_interleaved(part, positions, rot)
    else:
        angles = positions.double()[:, None] * freq[None, :]
        cos, sin = (torch.cos(angles) * magnitude)[:, None, :], (torch.sin(angles) * magnitude)[:, None, :]
        first, second = part[..., :rotary // 2], part[..., rotary // 2:]
        want = torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1)
    source = on_device(x)
    target = torch.zeros(tokens, heads, rotary + 2, dtype=dtype, device=device())
    table = on_device(freq.float())
    kernels.rope_rows(source[:, :, 4:4 + rotary], target[:, :, 2:], on_device(positions), table, magnitude, interleaved)
    close(target[:, :, 2:], want, max(tol, 2e-4), "rope_rows into another buffer")     # (angles are 32-bit products)
    assert float(target[:, :, :2].abs().max()) == 0.0
    kernels.rope_rows(source[:, :, 4:4 + rotary], source[:, :, 4:4 + rotary], on_device(positions), table, magnitude, interleaved)
    close(source[:, :, 4:4 + rotary], want, max(tol, 2e-4), "rope_rows in place")
    assert torch.equal(source[:, :, :4].cpu(), x[:, :, :4]) and torch.equal(source[:, :, 4 + rotary:].cpu(), x[:, :, 4 + rotary:])


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("q_rank,kv_rank,rotary", [(16, 24, 8), (5, 7, 2), (48, 64, 0), (300, 130, 64)])
def test_latents_are_normed_and_the_shared_key_part_rotated_into_the_cache(dtype, tol, q_rank, kv_rank, rotary):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(3)
    tokens, eps = 9, 1e-5
    q_offset, kv_offset = 8, 8 + -(-q_rank // 8) * 8
    packed = torch.randn(tokens, kv_offset + kv_rank + rotary + 3, generator=generator).to(dtype)
    q_norm, kv_norm = 1.0 + torch.randn(q_rank, generator=generator) * 0.3, 1.0 + torch.randn(kv_rank, generator=generator) * 0.3
    positions = torch.tensor([0, 1, 5, 16, 17, 100, 1000, 3, 2], dtype=torch.int32)
    slots = torch.tensor([4, 0, 9, -1, 2, 11, 7, 1, -1], dtype=torch.int32)
    rot = {"dims": rotary, "base": 10000.0, "scaling": {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}} if rotary else None
    freq, magnitude = plain.rotary_table(rot) if rotary else (torch.zeros(0, dtype=F64), 1.0)
    pages = torch.full((12, 1, kv_rank + rotary), 77.0, dtype=dtype, device=device())
    latent_q = torch.empty(tokens, q_rank, dtype=dtype, device=device())
    kernels.latent_prepare(on_device(packed), q_offset, q_rank, kv_offset, kv_rank, rotary, on_device(q_norm), on_device(kv_norm),
                           eps, on_device(positions), on_device(slots), on_device(freq.float()) if rotary else None, magnitude,
                           True, latent_q, pages)
    x = packed.double()
    close(latent_q, plain.unit_rms(x[:, q_offset:q_offset + q_rank], eps) * q_norm, tol, "query latent")
    latent = plain.unit_rms(x[:, kv_offset:kv_offset + kv_rank], eps) * kv_norm
    key = x[:, kv_offset + kv_rank:kv_offset + kv_rank + rotary]
    if rotary:
        key = plain.rotate_interleaved(key, positions, rot)
    want = torch.full((12, kv_rank + rotary), 77.0, dtype=F64)
    for token, slot in enumerate(slots.tolist()):
        if slot >= 0:
            want[slot] = torch.cat([latent[token], key[token]])
    close(pages[:, 0], want, max(tol, 2e-4) if rotary else tol, "cache rows (untouched where no token was written)")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("tokens,heads,in_dim,out_dim", [(1, 1, 8, 8), (9, 3, 20, 33), (70, 2, 300, 64), (17, 5, 7, 130)])
def test_a_product_per_head_with_and_without_gate(dtype, tol, tokens, heads, in_dim, out_dim):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(4)
    x = torch.randn(tokens, heads, in_dim + 5, generator=generator).to(dtype)
    w = (torch.randn(heads, in_dim, out_dim, generator=generator) * 0.3).to(dtype)
    gate = torch.randn(tokens, heads * out_dim + 8, generator=generator).to(dtype)
    want = torch.einsum("thi,hio->tho", x[:, :, 2:2 + in_dim].double(), w.double())
    out = torch.zeros(tokens, heads, out_dim + 3, dtype=dtype, device=device())
    kernels.head_linear(on_device(x)[:, :, 2:2 + in_dim], on_device(w), out[:, :, :out_dim])
    close(out[:, :, :out_dim], want, tol * 4, "head_linear")
    assert float(out[:, :, out_dim:].abs().max()) == 0.0
    gated = torch.empty(tokens, heads, out_dim, dtype=dtype, device=device())
    kernels.head_linear(on_device(x)[:, :, 2:2 + in_dim], on_device(w), gated, on_device(gate)[:, :heads * out_dim])
    close(gated, want * plain.sigmoid(gate[:, :heads * out_dim].double()).reshape(tokens, heads, out_dim), tol * 4, "head_linear, gated")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("page_size,rank,rotary", [(16, 24, 8), (8, 64, 16), (4, 20, 6), (32, 128, 0), (16, 512, 64)])
def test_attention_over_cached_latents_one_key_stands_out(dtype, tol, page_size, rank, rotary):
    """Every query is made to look at one chosen key: the first token, the one before and after a page border, a key
    hundreds of tokens back, the query's own.  The output must then be that key's latent; a kernel that loses a page,
    misreads the table or stops one key short gives another row."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(5)
    heads, width = 3, rank + rotary
    lengths = [1, page_size, page_size + 1, 5 * page_size - 1, 333, 700]
    pages_per = [-(-n // page_size) for n in lengths]
    order = torch.randperm(sum(pages_per) + 3, generator=generator).tolist()
    table = torch.full((len(lengths), max(pages_per)), -1, dtype=torch.int32)
    cache = torch.randn((sum(pages_per) + 3) * page_size, 1, width, generator=generator) * 50.0     # garbage elsewhere
    keys, cursor = [], 0
    for row, n in enumerate(lengths):
        k = torch.randn(n, width, generator=generator) * 0.3
        keys.append(k)
        for block in range(pages_per[row]):
            page = order[cursor]
            cursor += 1
            table[row, block] = page
            chunk = k[block * page_size:(block + 1) * page_size]
            cache[page * page_size:page * page_size + chunk.shape[0], 0] = chunk
    cache = cache.to(dtype)
    # one query per (request, target): the last position of the request looks at `target`
    queries, rows_of, positions, targets = [], [], [], []
    for row, n in enumerate(lengths):
        for target in sorted({0, n - 1, max(0, n - 2), min(n - 1, page_size - 1), min(n - 1, page_size), n // 2, max(0, n - 300)}):
            q = torch.randn(heads, width, generator=generator) * 0.1
            q[1] += keys[row][target] * 60.0                       # head 1 looks at the target, the others at everything
            queries.append(q)
            rows_of.append(row)
            positions.append(n - 1)
            targets.append(target)
    q = torch.stack(queries).to(dtype)
    out = torch.empty(len(queries), heads * rank, dtype=dtype, device=device())
    kernels.paged_attention_generic(on_device(q).view(len(queries), heads * width), out, on_device(cache), None, on_device(table),
                                    on_device(torch.tensor(rows_of, dtype=torch.int32)),
                                    on_device(torch.tensor(positions, dtype=torch.int32)), page_size, heads, 1, width, 0.5, None,
                                    value_dim=rank, values_in_keys=True)
    for index, (row, target) in enumerate(zip(rows_of, targets)):
        k = cache[:, 0].double()
        mine = torch.cat([k[table[row, b] * page_size:(table[row, b] + 1) * page_size] for b in range(pages_per[row])])[:lengths[row]]
        scores = torch.softmax((q[index].double() @ mine.T) * 0.5, dim=-1)
        want = scores @ mine[:, :rank]
        close(out[index].view(heads, rank), want, tol, f"request of {lengths[row]} keys, target {target}, page {page_size}")
        assert float(scores[1, target]) > 0.9


@pytest.mark.parametrize("partitions", [1, 3])
@pytest.mark.parametrize("heads,page_size,rank,rotary", [(3, 16, 24, 8), (16, 8, 64, 16), (5, 4, 128, 0), (16, 16, 512, 64),
                                                         (70, 32, 40, 8)])
def test_tensor_core_attention_over_cached_latents(heads, page_size, rank, rotary, partitions):
    """The tile kernel on single tokens beside prompt portions that start in the middle of a request, with shuffled
    pages and garbage in the rest of the pool: every (token, head) against a 64-bit softmax over the keys up to its
    own position; one head of every query is made to look at one far key."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(11)
    width = rank + rotary
    assert kernels.latent_attention_takes(width, rank)
    # (tokens in the step, tokens cached before it) per request row; single tokens first, as the engine packs them
    rows = [(1, 0), (1, 63), (1, 64), (1, 700), (2, 0), (65, 3), (130, 200), (17, 47)]
    contexts = [n + before for n, before in rows]
    pages_per = [-(-c // page_size) for c in contexts]
    order = torch.randperm(sum(pages_per) + 2, generator=generator).tolist()
    table = torch.full((len(rows), max(pages_per)), -1, dtype=torch.int32)
    cache = torch.randn((sum(pages_per) + 2) * page_size, 1, width, generator=generator) * 30.0
    keys, cursor = [], 0
    for row, context in enumerate(contexts):
        k = (torch.randn(context, width, generator=generator) * 0.4).to(torch.bfloat16).float()
        keys.append(k)
        for block in range(pages_per[row]):
            page = order[cursor]
            cursor += 1
            table[row, block] = page
            chunk = k[block * page_size:(block + 1) * page_size]
            cache[page * page_size:page * page_size + chunk.shape[0], 0] = chunk
    tokens = sum(n for n, _ in rows)
    q = torch.randn(tokens, heads, width, generator=generator) * 0.3
    starts, at = [0], 0
    for row, (n, before) in enumerate(rows):
        for i in range(n):
            target = (before + i) // 3                                      # a key well behind the query
            q[at + i, (at + i) % heads] += keys[row][target] * (40.0 / max(1.0, float(keys[row][target].norm()) ** 2) * 8.0)
        at += n
        starts.append(at)
    q = q.to(torch.bfloat16)
    out = torch.empty(tokens, heads * rank, dtype=torch.bfloat16, device=device())
    alloc = lambda shape, kind: torch.empty(shape, dtype=kind, device=device())
    longest = max(contexts)
    per_partition = -(-(-(-longest // 64)) // partitions) * 64
    kernels.latent_attention(on_device(q).view(tokens, heads * width), out, on_device(cache.to(torch.bfloat16)), on_device(table),
                             on_device(torch.tensor(starts, dtype=torch.int32)), on_device(torch.tensor(contexts, dtype=torch.int32)),
                             page_size, heads, width, rank, 0.5, max(n for n, _ in rows) * heads, per_partition,
                             -(-longest // per_partition), alloc)
    got = out.float().cpu().view(tokens, heads, rank)
    at = 0
    for row, (n, before) in enumerate(rows):
        k = keys[row].double()
        for i in range(n):
            visible = k[:before + i + 1]
            weights = torch.softmax((q[at + i].double() @ visible.T) * 0.5, dim=-1)
            close(got[at + i], weights @ visible[:, :rank], 2e-2, f"row {row}, token {i} of {n} after {before}")
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_blends_with_the_token_before_carry_over_portions(dtype):
    """wkv_mix: the token before a portion's first token is the request's state (zeros at its start); slots of other
    requests stay as they are; portions of one token and of several in one batch."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(6)
    width, slots = 52, 5
    mu = torch.rand(5, width, generator=generator)
    h = [torch.randn(n, width, generator=generator).to(dtype) for n in (13, 1, 6)]
    tail = torch.zeros(slots, width, device=device())
    tail[3] = 9.0                                                           # a slot nobody uses
    use = [2, 0, 4]
    cursors = [0, 0, 0]
    got = [[] for _ in h]
    for sizes in ([2, 1, 3], [1, 0, 1], [7, 0, 2], [3, 0, 0]):
        rows = [r for r, n in enumerate(sizes) if n]
        rows.sort(key=lambda r: sizes[r] != 1)                              # single-token rows first, as the engine packs
        packed = torch.cat([h[r][cursors[r]:cursors[r] + sizes[r]] for r in rows])
        description = batch_description([sizes[r] for r in rows], [use[r] for r in rows], [cursors[r] for r in rows])
        out = torch.empty(5, packed.shape[0], width, dtype=dtype, device=device())
        kernels.wkv_mix(on_device(packed), tail, on_device(mu), description[0], description[1], description[2], description[3], out,
                        single_tokens_only=all(sizes[r] == 1 for r in rows))
        at = 0
        for r in rows:
            got[r].append(out[:, at:at + sizes[r]].cpu())
            at += sizes[r]
            cursors[r] += sizes[r]
    for r, x in enumerate(h):
        x = x.double()
        before = torch.cat([torch.zeros(1, width, dtype=F64), x[:-1]])
        want = torch.stack([x + (before - x) * mu[s].double() for s in range(5)])
        close(torch.cat(got[r], dim=1), want, 2e-6 if dtype == torch.float32 else 8e-3, f"request {r}")
        close(tail[use[r]], x[-1], 0.0, "the state is the last input")
    assert float((tail[3] - 9.0).abs().max()) == 0.0 and float(tail[1].abs().max()) == 0.0


def plain_wkv_recurrence(r, k, v, decay, bonus, state):
    """r, k, v, decay [n, H, d]; bonus [H, d]; state [H, key, value] is updated in place; returns o [n, H, d]."""
    out = torch.zeros_like(v)
    for t in range(r.shape[0]):
        outer = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state + bonus[:, :, None] * outer, r[t])
        state.copy_(decay[t][:, :, None] * state + outer)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim", [(2, 64), (3, 20), (1, 128), (4, 6), (2, 100), (5, 32), (1, 160), (2, 256)])
def test_wkv_recurrence_against_the_plain_one(dtype, heads, dim):
    """The recurrence in portions with carried state, several requests in one launch (single tokens beside portions),
    other slots untouched; the inputs are the kernel's own (rounded) inputs, so the comparison is 32-bit sharp."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(7)
    width, slots = heads * dim, 4
    lengths = [45, 3, 20]
    inputs = []
    for n in lengths:
        r, k, v = (torch.randn(n, width, generator=generator).to(dtype) for _ in range(3))
        raw = torch.randn(n, width, generator=generator) - 1.0
        inputs.append((r, k, v, raw))
    bias, bonus = torch.randn(width, generator=generator) * 0.5, torch.randn(width, generator=generator) * 0.5
    state = torch.zeros(slots, heads, dim, dim, device=device())
    state[1] = 3.0
    use, cursors = [3, 0, 2], [0, 0, 0]
    got = [[] for _ in lengths]
    for sizes in ([1, 1, 1], [17, 1, 2], [1, 1, 16], [26, 0, 1]):
        rows = [i for i, n in enumerate(sizes) if n]
        rows.sort(key=lambda i: sizes[i] != 1)
        cut = lambda which: torch.cat([inputs[i][which][cursors[i]:cursors[i] + sizes[i]] for i in rows])
        description = batch_description([sizes[i] for i in rows], [use[i] for i in rows], [cursors[i] for i in rows])
        rkv = on_device(torch.stack([cut(0), cut(1), cut(2)]))
        out = torch.empty(rkv.shape[1], width, device=device())
        kernels.wkv_scan(rkv[0], rkv[1], rkv[2], on_device(cut(3)), on_device(bias), on_device(bonus), state, description[1],
                         description[2], description[3], out, heads, dim)
        at = 0
        for i in rows:
            got[i].append(out[at:at + sizes[i]].cpu())
            at += sizes[i]
            cursors[i] += sizes[i]
    for i, (r, k, v, raw) in enumerate(inputs):
        n = lengths[i]
        decay = torch.exp(-torch.exp(raw.double() + bias.double()))
        final = torch.zeros(heads, dim, dim, dtype=F64)
        shape = lambda x: x.double().reshape(n, heads, dim)
        want = plain_wkv_recurrence(shape(r), shape(k), shape(v), decay.reshape(n, heads, dim), bonus.double().reshape(heads, dim), final)
        close(torch.cat(got[i]), want.reshape(n, width), 2e-5, f"request {i}: read-out")
        close(state[use[i]].transpose(-1, -2), final, 2e-5, f"request {i}: state")          # (stored value channel first)
    assert float((state[1] - 3.0).abs().max()) == 0.0


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_head_norm_with_a_weight_per_head(dtype, tol):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(8)
    tokens, heads, dim = 7, 3, 20
    o = torch.randn(tokens, heads * dim, generator=generator) * 3.0
    gate = torch.randn(tokens, heads * dim, generator=generator).to(dtype)
    weight = 1.0 + torch.randn(heads * dim, generator=generator) * 0.3
    out = torch.empty(tokens, heads * dim, dtype=dtype, device=device())
    kernels.gated_head_norm(on_device(o), on_device(gate), on_device(weight), out, heads, dim, 1e-5, False)
    want = plain.unit_rms(o.double().reshape(tokens, heads, dim), 1e-5).reshape(tokens, -1) * weight * plain.silu(gate.double())
    close(out, want, tol, "gated_head_norm with [heads, dim] weights")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,groups,keep", [(8, 4, 2, 1), (6, 2, 3, 2), (4, 1, 1, 1), (12, 3, 12, 5), (9, 9, 1, 1), (16, 4, 4, 2)])
def test_router_against_the_plain_one(dtype, experts, top, groups, keep):
    """Choice scores that are negative (a large negative correction), groups of one expert, every expert chosen."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(9)
    tokens, width = 60, 52
    h = torch.randn(tokens, width, generator=generator).to(dtype)
    router = (torch.randn(experts, width, generator=generator) * 0.4).to(dtype)
    correction = torch.randn(experts, generator=generator) * 0.6 - 1.0
    gate_weight = (torch.randn(width, generator=generator) * 0.3).to(dtype)
    ids = torch.empty(tokens, top, dtype=torch.int32, device=device())
    weights = torch.empty(tokens, top, device=device())
    gate = torch.empty(tokens, device=device())
    stacked = torch.cat([router, gate_weight[None], torch.zeros(-(experts + 1) % 8, width, dtype=dtype)])
    logits = torch.empty(tokens, stacked.shape[0], device=device())
    kernels.linear(on_device(h), on_device(stacked), logits, alloc=lambda shape, kind: torch.empty(shape, dtype=kind, device=device()))
    kernels.moe_route(logits, on_device(correction), True, ids, weights, gate, experts, top, groups, keep, 2.5)
    table = {"m.router": router.double(), "m.correction": correction.double()}
    chosen, share = plain.route(h.double(), table, "m.", {"experts": experts, "top": top, "scale": 2.5,
                                                         "groups": {"count": groups, "keep": keep}})
    got_ids, got_weights = ids.cpu().long(), weights.cpu().double()
    for t in range(tokens):
        assert sorted(got_ids[t].tolist()) == sorted(chosen[t].tolist()), f"token {t}"
        by_expert = dict(zip(chosen[t].tolist(), share[t].tolist()))
        for expert, weight in zip(got_ids[t].tolist(), got_weights[t].tolist()):
            assert abs(weight - by_expert[expert]) <= 2e-5 * 2.5
    close(gate, plain.sigmoid(h.double() @ gate_weight.double()), 1e-5, "the shared expert's gate")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("tokens,experts,top,width,inter", [(1, 4, 2, 32, 16), (7, 3, 3, 52, 20), (100, 16, 4, 64, 40),
                                                            (33, 5, 1, 600, 24), (9, 40, 2, 24, 7), (300, 3, 2, 72, 136),
                                                            (700, 5, 3, 264, 200)])
def test_experts_on_ordered_pairs_against_token_by_token(dtype, tol, tokens, experts, top, width, inter):
    """Sorting by expert, the two grouped products (32-bit multiply-adds on tiles of 8 pairs, or the tcgen05 product
    on tiles of 128 where the sizes allow) and the weighted sum: experts without any token, experts with more pairs than
    a tile, a shared expert with and without gate."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(10)
    h = torch.randn(tokens, width, generator=generator).to(dtype)
    both = (torch.randn(2 * experts, inter, width, generator=generator) * 0.2).to(dtype)
    w_gate, w_up = both[:experts], both[experts:]
    w_down = (torch.randn(experts, width, inter, generator=generator) * 0.2).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=generator)[:top] for _ in range(tokens)]).to(torch.int32)
    if top == 1 and experts > 2:
        ids[ids == 1] = 0                                                    # expert 1 gets no token
    weights = torch.rand(tokens, top, generator=generator)
    alloc = lambda shape, kind: torch.empty(shape, dtype=kind, device=device())
    tile = kernels.expert_tile_pairs(dtype, width, inter)
    assert tile == (128 if dtype == torch.bfloat16 and width % 8 == 0 and inter % 8 == 0 else 8)
    found = kernels.moe_sort(on_device(ids), experts, alloc, tile)
    order, offsets = found.order.cpu().tolist(), found.offsets.cpu().tolist()
    flat = ids.reshape(-1).tolist()
    assert sorted(order) == list(range(tokens * top)) and offsets[0] == 0 and offsets[-1] == tokens * top
    for expert in range(experts):
        mine = order[offsets[expert]:offsets[expert + 1]]
        assert all(flat[pair] == expert for pair in mine) and mine == sorted(mine)
    tiles = found.tiles.cpu().tolist()
    count = int(found.tile_count.cpu())
    covered = []
    for n in range(count):
        expert, start = tiles[2 * n], tiles[2 * n + 1]
        covered += list(range(start, min(start + tile, offsets[expert + 1])))
        assert offsets[expert] <= start < offsets[expert + 1]
    assert sorted(covered) == list(range(tokens * top))
    hidden = torch.empty(tokens * top, inter, dtype=dtype, device=device())
    both = on_device(both)
    kernels.moe_gate_up(on_device(h), found, top, both[:experts], both[experts:], hidden, alloc)
    pair_rows = torch.empty(tokens * top, width, device=device())
    kernels.moe_down(hidden, found, on_device(w_down), pair_rows)
    shared = torch.randn(tokens, width, generator=generator)
    gate = torch.rand(tokens, generator=generator)
    want = torch.zeros(tokens, width, dtype=F64)
    for t in range(tokens):
        for slot in range(top):
            e = int(ids[t, slot])
            x = h[t].double()
            inner = plain.silu(w_gate[e].double() @ x) * (w_up[e].double() @ x)
            if dtype == torch.bfloat16:
                inner = inner.to(torch.bfloat16).double()                  # (the hidden rows are stored in 16 bits)
            want[t] += float(weights[t, slot]) * (w_down[e].double() @ inner)
    base = torch.randn(tokens, width, generator=generator)
    for rows, gates, extra in ((None, None, 0), (shared, gate, shared.double() * gate.double()[:, None]), (shared, None, shared.double())):
        residual = on_device(base.clone())
        kernels.moe_combine(residual, pair_rows, on_device(weights), on_device(rows) if rows is not None else None,
                            on_device(gates) if gates is not None else None)
        close(residual, base.double() + want + extra, tol, f"{tokens} tokens, {experts} experts, top {top}")
    if dtype == torch.bfloat16:
        assert kernels.tensor_core_linear_error() == 0


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


def test_the_residual_stream_after_every_layer_run(tmp_path):
    """One prompt in 32-bit: the residual after each run of a layer (looped layers count each time) against the
    plain implementation's, so that a fault shows at the layer that has it."""
    from libmir_b200 import StepEntry
    from libmir_b200.parts.block import ParallelBlock
    config = ALL["A"]
    folder = make_folder(tmp_path, config, seed=2, dtype="float32")
    ids = random_ids(np.random.default_rng(1), config["vocab"], 40)
    plain_config, weights = plain.read_model(folder)
    want = []
    plain.forward(plain_config, weights, ids, want)
    model = load(folder, "float32", 8, 16)
    seen, original = [], ParallelBlock.forward

    def recording(self, ctx, cache, residual):
        original(self, ctx, cache, residual)
        seen.append(residual.clone())
    ParallelBlock.forward = recording
    try:
        model.admit("x")
        model.step([StepEntry("x", ids, [0])])
    finally:
        ParallelBlock.forward = original
    assert len(seen) == len(want) == len(plain.layer_order(config))
    for run, (got, expected) in enumerate(zip(seen, want)):
        close(got, expected, 2e-5, f"after layer run {run} (layer {plain.layer_order(config)[run][0]})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole_prompts_token_by_token_and_portions(tmp_path, name, dtype):
    """A prompt whole; the same token by token from its first token (150 single steps: long decoding, keys that get
    far away, the first tokens of a sequence); and in portions of changing size down to two tokens."""
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
        # reduces a query's keys in an order that depends on its position alone, products reduce in one fixed order
        assert np.array_equal(whole, single) and np.array_equal(whole, portions) and np.array_equal(whole, late)
    for group in model.cache_stats()["groups"]:
        assert group["free"] == group["pages"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
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
    if dtype == "float32":
        for index in range(len(requests)):
            close_logits(np.concatenate(got[index]), want[index], dtype, f"{name}/{dtype} request {index} in a mixed batch")
    else:       # (the share of positions is taken over all requests: the shortest has eighteen)
        close_logits(np.concatenate([np.concatenate(got[index]) for index in range(len(requests))]), np.concatenate(want),
                     dtype, f"{name}/{dtype} requests in mixed batches")
    stats = model.cache_stats()
    assert stats["free_slots"] == 3
    for group in stats["groups"]:
        assert group["free"] == group["pages"] and group["reused"] > 0


def test_a_far_key_decides_the_logits_in_prompt_and_in_decoding(tmp_path):
    """One layer of latent attention whose queries are sharp: the logits at the last positions depend on keys hundreds
    of tokens back, over many pages; whole, and with the last tokens decoded one by one."""
    config = {"architecture": "Zufotar", "vocab": 90, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 24, "q_rank": 32, "kv_rank": 40, "scale": 0.25,
                   "rot": {"dims": 8, "base": 10000.0, "scaling": {"factor": 2.0, "original": 128, "fast": 16.0, "slow": 1.0}}}}]}
    rng = np.random.default_rng(4)
    ids = random_ids(rng, 90, 700)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=6, dtype=dtype, sharpen=30.0)
        plain_config, weights = plain.read_model(folder)
        want = plain.forward(plain_config, weights, ids).numpy()
        shorter = plain.forward(plain_config, weights, ids[300:]).numpy()
        # the early keys matter: without the first 300 tokens the last logits are others
        assert np.abs(shorter[-20:] - want[-20:]).max() > 0.1
        model = load(folder, dtype, 16, 50)
        close_logits(feed(model, "whole", ids, [700]), want, dtype, f"far keys, whole, {dtype}")
        close_logits(feed(model, "late", ids, [650, 1]), want, dtype, f"far keys, decoded, {dtype}")
        close_logits(feed(model, "cut", ids, [15, 17, 300, 2, 31]), want, dtype, f"far keys, portions, {dtype}")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "B"])
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


def test_decode_steps_replayed_from_captured_graphs_in_bfloat16(tmp_path):
    """Two requests decoded together through captured graphs in bfloat16 (the tensor-core attention kernel with its
    keys split, the experts on the tcgen05 product with its tiles read from the device): the teacher-forced logits of
    every step against the plain implementation."""
    from libmir_b200 import StepEntry, kernels
    from libmir_b200.sampling import RequestSampler
    config = ALL["A"]
    folder = make_folder(tmp_path, config, seed=8, dtype="bfloat16")
    rng = np.random.default_rng(5)
    requests = {"a": random_ids(rng, config["vocab"], 60), "b": random_ids(rng, config["vocab"], 47)}
    want = {name: reference(folder, ids) for name, ids in requests.items()}
    prompt = {"a": 21, "b": 8}
    model = load(folder, "bfloat16", 8, 40, graphs=True)
    got = {name: [] for name in requests}
    for name, ids in requests.items():
        model.admit(name)
        result = model.step([StepEntry(name, ids[:prompt[name]], range(prompt[name]))])
        got[name].append(result.logits.float().cpu().numpy().copy())
    for step in range(39):
        entries = [StepEntry(name, [ids[prompt[name] + step]], [0]) for name, ids in requests.items()]
        result = model.step(entries, [RequestSampler() for _ in entries])
        logits = result.logits.float().cpu().numpy()
        for row, name in enumerate(requests):
            got[name].append(logits[row:row + 1].copy())
    assert model.runner._graphs is not None and len(model.runner._graphs.graphs) > 0
    everything = np.concatenate([np.concatenate(got[name]) for name in requests])
    wanted = np.concatenate([want[name][:prompt[name] + 39] for name in requests])
    close_logits(everything, wanted, "bfloat16", "decode steps from captured graphs")
    assert kernels.tensor_core_linear_error() == 0


def test_trace_runner_picks_the_design_by_its_configuration(tmp_path):
    """bin/trace_run as a user runs it: the model class comes from config.json; prompts in portions, decoded tokens,
    a pool that holds less than all requests together."""
    config = ALL["C"]
    folder = make_folder(tmp_path / "model", config, seed=4, dtype="bfloat16")
    (folder / "config.json").write_text(json.dumps(dict(config, vocab_size=config["vocab"])))   # (helpers read this key)
    rng = np.random.default_rng(3)
    requests = {f"q{i}": random_ids(rng, config["vocab"], n) for i, n in enumerate((100, 64, 37))}
    want = {name: reference(folder, ids) for name, ids in requests.items()}
    # (the third run replays every single-token step from a captured graph, as generation does)
    for dtype, extra in (("bfloat16", []), ("float32", []), ("bfloat16", ["--decode-graphs"])):
        trace = Trace()
        for name, ids in requests.items():
            trace.step([(name, ids[:len(ids) - 10], [0, len(ids) - 11])])
            for position in range(len(ids) - 10, len(ids)):
                trace.step([(name, ids[position:position + 1], [0])], end=[name] if position == len(ids) - 1 else [])
        results = run_trace(folder, dtype, trace, tmp_path / f"out-{dtype}-{len(extra)}", max_tokens=128,
                            extra_args=["--page-size", "8"] + extra)
        got = np.stack([results[index][row] for index, rows in enumerate(trace.expect) for row in range(len(rows))])
        wanted = np.stack([want[name][position] for rows in trace.expect for name, position in rows])
        close_logits(got, wanted, dtype, f"trace {dtype} {extra}")


def test_generate_command_line(tmp_path):
    """bin/generate on a model folder of the design: two prompts as one batch, greedy, against the plain
    implementation."""
    import subprocess
    import sys
    from helpers import ROOT
    config = ALL["D"]
    folder = make_folder(tmp_path / "model", config, seed=12, dtype="float32")
    plain_config, weights = plain.read_model(folder)
    command = [sys.executable, str(ROOT / "bin" / "generate"), str(folder), "--dtype", "float32", "--block-size", "8",
               "--block-count", "64", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(command + ["--prompt-ids", "5,9,80,33;7", "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    outputs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(outputs) == 2
    for prompt, output in zip(([5, 9, 80, 33], [7]), outputs):
        ids = list(prompt)
        for token in output["token_ids"]:
            logits = plain.forward(plain_config, weights, ids)[-1]
            best = int(torch.argmax(logits))
            assert token == best or float(logits[best] - logits[token]) < 1e-4
            ids.append(token)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes nobody chose: a prompt whole, token by token, in portions and as a prompt followed by decoding, in both
    dtypes, against the plain implementation (32-bit: every position within 2e-4 of its logits' root mean square and
    the same bits under every cut; bfloat16: nine positions in ten within the tolerance)."""
    rng = np.random.default_rng(700 + seed)
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
