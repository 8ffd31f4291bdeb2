"""Each kernel alone against its plain statement (tests/plain_ops.py, computed in float64),
at sizes other than the engine's: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head counts and groups, page sizes from 1 up."""

from __future__ import annotations

import struct

import pytest
import torch

import plain_ops
import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def kernels():
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels as k
    k.library()
    return k


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [1, 48, 72, 1000, 2048, 5120])
def test_embedding(kernels, dtype, hidden):
    table = rand((331, hidden), dtype, 1)
    tokens = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32).cuda()
    out = torch.empty((5, hidden), dtype=torch.float32).cuda()
    kernels.embedding(tokens, table, out)
    assert torch.equal(out, table[tokens.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("weight_dtype", DTYPES)
@pytest.mark.parametrize("hidden,eps", [(1, 1e-6), (31, 1e-5), (72, 1e-6), (257, 1e-3), (1031, 1e-6), (2048, 1e-6), (4096, 1e-6),
                                        (6144, 1e-5), (8192, 1e-6), (8200, 1e-6)])
def test_add_rmsnorm(kernels, dtype, weight_dtype, hidden, eps):
    if dtype == torch.float32 and weight_dtype == torch.bfloat16:
        pytest.skip("a float32 model keeps float32 weights")
    n = 7
    residual = rand((n, hidden), torch.float32, 2, 3.0)
    delta = rand((n, hidden), dtype, 3)
    weight = (1 + rand((hidden,), torch.float32, 4, 0.1)).to(weight_dtype)
    expected_res = residual.double() + delta.double()
    expected = torch.empty((n, hidden), dtype=torch.float64).cuda()
    plain_ops.add_rmsnorm(residual.clone().double(), delta, weight, eps, expected)
    out = torch.empty((n, hidden), dtype=dtype).cuda()
    kernels.add_rmsnorm(residual, delta, weight, eps, out)
    assert torch.allclose(residual.double(), expected_res, atol=1e-6, rtol=1e-6)
    assert torch.allclose(out.double(), expected, **tol(dtype))
    # gathered rows, residual untouched; and no delta
    rows = torch.tensor([6, 0, 3], dtype=torch.int32).cuda()
    before = residual.clone()
    out_rows = torch.empty((3, hidden), dtype=dtype).cuda()
    kernels.add_rmsnorm(residual, delta, weight, eps, out_rows, rows)
    assert torch.equal(residual, before)
    expected_rows = torch.empty((3, hidden), dtype=torch.float64).cuda()
    plain_ops.add_rmsnorm(residual.double(), delta, weight, eps, expected_rows, rows)
    assert torch.allclose(out_rows.double(), expected_rows, **tol(dtype))
    out_plain = torch.empty((n, hidden), dtype=dtype).cuda()
    kernels.add_rmsnorm(residual, None, weight, eps, out_plain)
    assert torch.equal(residual, before)
    expected_plain = torch.empty((n, hidden), dtype=torch.float64).cuda()
    plain_ops.add_rmsnorm(residual.double(), None, weight, eps, expected_plain)
    assert torch.allclose(out_plain.double(), expected_plain, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [16, 48, 128, 200])
def test_rmsnorm_rows(kernels, dtype, size):
    x = rand((5, 3, size), dtype, 5, 2.0)
    weight = (1 + rand((size,), torch.float32, 6, 0.1)).to(dtype)
    out = torch.empty_like(x)
    kernels.rmsnorm(x, weight, 1e-5, out)
    expected = torch.empty(x.shape, dtype=torch.float64).cuda()
    plain_ops.rmsnorm(x, weight, 1e-5, expected)
    assert torch.allclose(out.double(), expected, **tol(dtype))


@pytest.mark.parametrize("half,theta", [(8, 1e4), (24, 5e4), (64, 1e6)])
def test_rope_table(kernels, half, theta):
    positions = torch.tensor([0, 1, 2, 77, 4095, 40959], dtype=torch.int32).cuda()
    inv_freq = (1.0 / (theta ** (torch.arange(0, 2 * half, 2, dtype=torch.float32) / (2 * half)))).cuda()
    table = torch.empty((6, half, 2), dtype=torch.float32).cuda()
    kernels.rope_table(positions, inv_freq, table)
    expected = torch.empty((6, half, 2), dtype=torch.float64).cuda()
    plain_ops.rope_table(positions, inv_freq, expected)
    assert torch.allclose(table.double(), expected, atol=3e-7, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,rotary,interleaved,with_norm", [
    (4, 2, 16, 16, 16, False, True), (6, 2, 32, 8, 32, False, True), (3, 1, 48, 4, 48, False, True),
    (5, 5, 64, 1, 32, False, True), (8, 2, 128, 64, 128, True, False), (2, 1, 256, 3, 64, True, True),
    (4, 4, 80, 16, 0, False, True)])
def test_qk_norm_rope_append(kernels, dtype, n_q, n_kv, d, page_size, rotary, interleaved, with_norm):
    n, pages = 11, 16
    qkv = rand((n, (n_q + 2 * n_kv) * d), dtype, 7)
    q_w = (1 + rand((d,), torch.float32, 8, 0.1)).to(dtype) if with_norm else None
    k_w = (1 + rand((d,), torch.float32, 9, 0.1)).to(dtype) if with_norm else None
    positions = torch.tensor([3, 4, 5, 0, 100, 101, 102, 103, 104, 9, 10], dtype=torch.int32).cuda()
    g = torch.Generator().manual_seed(10)
    slots = torch.randperm(pages * page_size, generator=g)[:n].to(torch.int32)
    slots[4] = -1
    slots = slots.cuda()
    cos_sin = None
    if rotary:
        inv_freq = (1.0 / (1e4 ** (torch.arange(0, rotary, 2, dtype=torch.float32) / rotary))).cuda()
        cos_sin = torch.empty((n, rotary // 2, 2), dtype=torch.float32).cuda()
        kernels.rope_table(positions, inv_freq, cos_sin)
    k_pool = torch.zeros((pages, n_kv, page_size, d), dtype=dtype).cuda()
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty((n, n_q, d), dtype=dtype).cuda()
    kernels.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, rotary, interleaved, k_pool, v_pool, n_q, n_kv, d, q_out)
    ek, ev = torch.zeros(k_pool.shape, dtype=torch.float64).cuda(), torch.zeros(k_pool.shape, dtype=torch.float64).cuda()
    eq = torch.empty(q_out.shape, dtype=torch.float64).cuda()
    plain_ops.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, rotary, interleaved, ek, ev, n_q, n_kv, d, eq)
    assert torch.allclose(q_out.double(), eq, **tol(dtype))
    assert torch.allclose(k_pool.double(), ek, **tol(dtype))
    assert torch.equal(v_pool.double(), ev)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,n", [(16, 8, 128, 64, 600), (8, 2, 64, 16, 1500), (4, 4, 32, 8, 1377), (3, 1, 16, 4, 3300)])
def test_qk_norm_rope_append_of_many_tokens(kernels, dtype, n_q, n_kv, d, page_size, n):
    """Prompt portions: thousands of (token, head) pairs, a number of them that is no multiple of what a block
    takes, tokens without a slot, and every head size with a power-of-two number of lanes."""
    pages = (n + page_size - 1) // page_size + 2
    qkv = rand((n, (n_q + 2 * n_kv) * d), dtype, 17)
    q_w, k_w = (1 + rand((d,), torch.float32, 18, 0.1)).to(dtype), (1 + rand((d,), torch.float32, 19, 0.1)).to(dtype)
    g = torch.Generator().manual_seed(20)
    positions = torch.randint(0, 5000, (n,), generator=g).to(torch.int32).cuda()
    slots = torch.randperm(pages * page_size, generator=g)[:n].to(torch.int32)
    slots[::97] = -1
    slots = slots.cuda()
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    cos_sin = torch.empty((n, d // 2, 2), dtype=torch.float32).cuda()
    kernels.rope_table(positions, inv_freq, cos_sin)
    k_pool = torch.zeros((pages, n_kv, page_size, d), dtype=dtype).cuda()
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty((n, n_q, d), dtype=dtype).cuda()
    kernels.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, d, False, k_pool, v_pool, n_q, n_kv, d, q_out)
    ek, ev = torch.zeros(k_pool.shape, dtype=torch.float64).cuda(), torch.zeros(k_pool.shape, dtype=torch.float64).cuda()
    eq = torch.empty(q_out.shape, dtype=torch.float64).cuda()
    plain_ops.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, d, False, ek, ev, n_q, n_kv, d, eq)
    assert torch.allclose(q_out.double(), eq, **tol(dtype))
    assert torch.allclose(k_pool.double(), ek, **tol(dtype))
    assert torch.equal(v_pool.double(), ev)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,paired", [(1, False), (200, False), (224, False), (6144, False), (8, True), (200, True), (6144, True)])
def test_silu_mul(kernels, dtype, inter, paired):
    gate_up = rand((5, 2 * inter), dtype, 11, 3.0)
    out = torch.empty((5, inter), dtype=dtype).cuda()
    kernels.silu_mul(gate_up, out, paired=paired)
    expected = torch.empty((5, inter), dtype=torch.float64).cuda()
    plain_ops.silu_mul(gate_up, expected, paired=paired)
    assert torch.allclose(out.double(), expected, **tol(dtype))


def test_silu_mul_refuses_paired_columns_of_a_ragged_size(kernels):
    gate_up = rand((2, 2 * 12), torch.float32, 11)
    with pytest.raises(kernels.KernelError, match="multiple of 8"):
        kernels.silu_mul(gate_up, torch.empty((2, 12)).cuda(), paired=True)


def _attention_case(dtype, n_q, n_kv, d, page_size, lengths, query_lens, seed):
    """Requests with context ``lengths`` whose last ``query_lens`` tokens are the step's queries;
    pages are handed out in a shuffled order so that tables are neither contiguous nor sorted."""
    g = torch.Generator().manual_seed(seed)
    pages_needed = [(n + page_size - 1) // page_size for n in lengths]
    total = sum(pages_needed) + 3
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages_needed)
    tables, cursor = [], 0
    for need in pages_needed:
        tables.append(order[cursor:cursor + need] + [total - 1] * (width - need))
        cursor += need
    k_pool = rand((total, n_kv, page_size, d), dtype, seed + 1)
    v_pool = rand((total, n_kv, page_size, d), dtype, seed + 2)
    request_of_token, positions, query_start = [], [], [0]
    for r, (length, q_len) in enumerate(zip(lengths, query_lens)):
        request_of_token += [r] * q_len
        positions += list(range(length - q_len, length))
        query_start.append(len(positions))
    n = len(positions)
    q = rand((n, n_q, d), dtype, seed + 3)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    return (q, k_pool, v_pool, as_int(tables), as_int(request_of_token), as_int(positions), as_int(query_start),
            as_int(lengths), max(query_lens), max(lengths))


@pytest.mark.parametrize("dtype", DTYPES)
def _check_attention(kernels, dtype, case, d, window, with_host_lengths=False):
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q, max_ctx = case
    out = torch.empty_like(q)
    kernels.paged_attention(q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                            max_ctx, d ** -0.5, window, out, query_start.tolist() if with_host_lengths else None)
    kernels.check_device_errors(q.device)
    expected = torch.empty(q.shape, dtype=torch.float64).cuda()
    plain_ops.paged_attention(q.cpu(), k_pool.cpu(), v_pool.cpu(), tables.cpu(), request_of_token.cpu(), positions.cpu(),
                              query_start.cpu(), context_lens.cpu(), max_q, max_ctx, d ** -0.5, window, expected)
    assert torch.allclose(out.double(), expected, **tol(dtype)), float((out.double() - expected).abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,window", [
    (4, 2, 16, 16, None), (6, 2, 32, 8, None), (3, 1, 48, 4, None), (5, 5, 64, 1, None), (8, 1, 128, 64, None),
    (2, 2, 256, 16, None), (4, 2, 80, 5, 7), (6, 3, 96, 16, 33), (4, 1, 112, 32, 1), (16, 8, 128, 16, None),
    (6, 1, 64, 16, 50), (4, 2, 128, 3, 20), (40, 2, 32, 16, None)])
def test_paged_attention(kernels, dtype, n_q, n_kv, d, page_size, window):
    """Portions of prompts (down to one token) beside each other: every kernel variant, shuffled pages."""
    lengths, query_lens = [1, 37, 130, 64, 200, 333], [1, 5, 1, 64, 2, 333]
    _check_attention(kernels, dtype, _attention_case(dtype, n_q, n_kv, d, page_size, lengths, query_lens, 20), d, window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,window", [
    (16, 8, 128, 16, None), (6, 2, 32, 8, None), (8, 1, 64, 5, None), (4, 4, 128, 64, 100), (48, 2, 64, 16, None)])
def test_paged_attention_decode_steps(kernels, dtype, n_q, n_kv, d, page_size, window):
    """Single tokens only, so that the keys are split over several thread blocks and merged."""
    lengths = [1, 2, 31, 32, 33, 700, 1500]
    _check_attention(kernels, dtype, _attention_case(dtype, n_q, n_kv, d, page_size, lengths, [1] * len(lengths), 21), d, window)
    lengths = [2500]
    _check_attention(kernels, dtype, _attention_case(dtype, n_q, n_kv, d, page_size, lengths, [1], 22), d, window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,window", [(16, 8, 128, 16, None), (8, 2, 64, 64, None), (6, 2, 32, 8, 40), (4, 4, 48, 4, None)])
def test_paged_attention_single_tokens_before_portions(kernels, dtype, n_q, n_kv, d, page_size, window):
    """A mixed step as the scheduler builds it: decoded tokens first, then prompt portions (two launches)."""
    lengths, query_lens = [700, 1500, 1, 64, 333], [1, 1, 1, 64, 300]
    _check_attention(kernels, dtype, _attention_case(dtype, n_q, n_kv, d, page_size, lengths, query_lens, 23), d, window,
                     with_host_lengths=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("query_len", [3, 1])
def test_paged_attention_finds_one_far_key(kernels, dtype, query_len):
    """One key among hundreds is made to dominate; the output must be (almost) its value row."""
    n_q, n_kv, d, page_size = 4, 2, 64, 16
    lengths, query_lens = [700], [query_len]
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q, max_ctx = \
        _attention_case(dtype, n_q, n_kv, d, page_size, lengths, query_lens, 30)
    for target in (0, 15, 16, 300, 696):
        kp = k_pool.clone()
        page, offset = int(tables[0, target // page_size]), target % page_size
        for head in range(n_kv):
            kp[page, head, offset] = (q[0, head * 2].float() * 40).to(dtype)
        out = torch.empty_like(q)
        kernels.paged_attention(q, kp, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                                max_ctx, d ** -0.5, None, out)
        for head in (0, 2):
            assert torch.allclose(out[0, head].float(), v_pool[page, head // 2, offset].float(), atol=2e-2), target


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("query_len", [1, 4])
@pytest.mark.parametrize("d", [64, 48])
def test_paged_attention_window_edge(kernels, dtype, query_len, d):
    """A dominant key just outside the window must be invisible, just inside it must win."""
    n_q, n_kv, page_size, window, length = 2, 1, 16, 37, 200
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q, max_ctx = \
        _attention_case(dtype, n_q, n_kv, d, page_size, [length], [query_len], 31)
    last = length - 1                                   # position of the last query token
    for key, visible in ((last - window, False), (last - window + 1, True), (last, True)):
        kp = k_pool.clone()
        page, offset = int(tables[0, key // page_size]), key % page_size
        kp[page, 0, offset] = (q[query_len - 1, 0].float() * 40).to(dtype)
        out = torch.empty_like(q)
        kernels.paged_attention(q, kp, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                                max_ctx, d ** -0.5, window, out)
        close = torch.allclose(out[query_len - 1, 0].float(), v_pool[page, 0, offset].float(), atol=3e-2)
        assert close == visible, (key, visible)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page_size,window,softcap,slopes", [
    (4, 2, 64, 16, None, 5.0, False), (8, 2, 128, 8, None, None, True), (6, 3, 48, 4, 21, 2.5, True), (2, 1, 24, 16, None, 30.0, True)])
def test_paged_attention_score_modifiers(kernels, dtype, n_q, n_kv, d, page_size, window, softcap, slopes):
    """A soft cap on the scores and a bias that grows with the distance between query and key (one slope per
    query head), which only the general kernel implements: sizes that would otherwise run on tensor cores too."""
    lengths, query_lens = [1, 37, 130, 200], [1, 5, 1, 64]
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q, max_ctx = \
        _attention_case(dtype, n_q, n_kv, d, page_size, lengths, query_lens, 35)
    bias = torch.tensor([0.5 ** (1 + h) for h in range(n_q)], dtype=torch.float32).cuda() if slopes else None
    out = torch.empty_like(q)
    kernels.paged_attention(q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                            max_ctx, d ** -0.5, window, out, None, softcap, bias)
    expected = torch.empty(q.shape, dtype=torch.float64)
    plain_ops.paged_attention(q.cpu(), k_pool.cpu(), v_pool.cpu(), tables.cpu(), request_of_token.cpu(), positions.cpu(),
                              query_start.cpu(), context_lens.cpu(), max_q, max_ctx, d ** -0.5, window, expected,
                              None, softcap, None if bias is None else bias.cpu())
    assert torch.allclose(out.double().cpu(), expected, **tol(dtype)), float((out.double().cpu() - expected).abs().max())
    plain = torch.empty_like(q)
    kernels.paged_attention(q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                            max_ctx, d ** -0.5, window, plain)
    assert not torch.allclose(out.float(), plain.float(), atol=1e-2)      # the modifiers did change something


def test_embedding_scale_and_logit_transform(kernels):
    table = rand((50, 72), torch.bfloat16, 60)
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32).cuda()
    out = torch.empty((4, 72), dtype=torch.float32).cuda()
    kernels.embedding(tokens, table, out, 8.5)
    assert torch.equal(out, 8.5 * table[tokens.long()].float())
    logits = rand((3, 331), torch.float32, 61, 20.0)
    expected = 30.0 * torch.tanh(0.25 * logits.double() / 30.0)
    kernels.scale_softcap(logits, 0.25, 30.0)
    assert torch.allclose(logits.double(), expected, atol=1e-5, rtol=1e-5)
    only_scaled = rand((2, 17), torch.float32, 62)
    before = only_scaled.clone()
    kernels.scale_softcap(only_scaled, 3.0)
    assert torch.equal(only_scaled, 3.0 * before)


@pytest.mark.parametrize("n_q,n_kv,d,page_size,window,with_norm,with_rope,weight_dtype", [
    (16, 8, 128, 64, None, True, True, torch.bfloat16), (8, 2, 64, 16, None, True, True, torch.float32),
    (6, 1, 128, 8, 300, False, True, torch.bfloat16), (4, 4, 64, 32, 70, True, False, torch.bfloat16),
    (32, 2, 128, 16, None, True, True, torch.float32)])
@pytest.mark.parametrize("lengths", [[1, 2, 31, 32, 33, 700, 1500], [2500], [129] * 9, [64, 4000] * 20])
def test_decode_attention_with_norm_rotation_and_append_inside(kernels, lengths, n_q, n_kv, d, page_size, window, with_norm,
                                                               with_rope, weight_dtype):
    """A decode step's norm + rotation + append inside the split-key attention kernel, against the plain versions of
    the separate steps: the attended heads, and what the cache holds afterwards.  One to many splits, requests of
    one key, windows, a request whose key is in the cache already (no slot), and a dominant far key."""
    dtype = torch.bfloat16
    n = len(lengths)
    assert kernels.decode_attention_fused_supported(dtype, d, n_q, n_kv)
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, _, max_ctx = \
        _attention_case(dtype, n_q, n_kv, d, page_size, lengths, [1] * n, 41)
    qkv = rand((n, (n_q + 2 * n_kv) * d), dtype, 42)
    q_w = (1 + rand((d,), torch.float32, 43, 0.1)).to(weight_dtype) if with_norm else None
    k_w = (1 + rand((d,), torch.float32, 44, 0.1)).to(weight_dtype) if with_norm else None
    cos_sin = None
    if with_rope:
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
        cos_sin = torch.empty((n, d // 2, 2), dtype=torch.float32).cuda()
        kernels.rope_table(positions, inv_freq, cos_sin)
    slots = torch.tensor([int(tables[r, (length - 1) // page_size]) * page_size + (length - 1) % page_size
                          for r, length in enumerate(lengths)], dtype=torch.int32)
    if n > 2:
        slots[2] = -1                      # this request's newest key and value are in the cache already
    slots = slots.cuda()
    # the plain steps, on copies of the cache
    ek, ev = k_pool.double().clone(), v_pool.double().clone()
    eq = torch.empty((n, n_q, d), dtype=torch.float64).cuda()
    plain_ops.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, d if with_rope else 0, False, ek, ev, n_q, n_kv, d, eq)
    dominated = None
    if lengths[-1] > 600:                  # one old key of the last request is made to dominate its first query head
        target = lengths[-1] - 500 if window is None else lengths[-1] - window + 3
        page, offset = int(tables[n - 1, target // page_size]), target % page_size
        k_pool[page, 0, offset] = (eq[n - 1, 0] * 40).to(dtype)
        ek[page, 0, offset] = k_pool[page, 0, offset].double()
        dominated = (page, offset)
    expected = torch.empty((n, n_q, d), dtype=torch.float64)
    plain_ops.paged_attention(eq.to(dtype).cpu(), ek.to(dtype).cpu(), ev.to(dtype).cpu(), tables.cpu(), request_of_token.cpu(),
                              positions.cpu(), query_start.cpu(), context_lens.cpu(), 1, max_ctx, d ** -0.5, window, expected)
    out = torch.full((n, n_q, d), 7.0, dtype=dtype).cuda()
    kernels.decode_attention_fused(qkv, slots, q_w, k_w, 1e-6, cos_sin, k_pool, v_pool, tables, query_start, context_lens,
                                   max_ctx, d ** -0.5, window, n_q, n_kv, d, out)
    torch.cuda.synchronize()
    assert torch.allclose(out.double().cpu(), expected, atol=2e-2, rtol=2e-2), float((out.double().cpu() - expected).abs().max())
    assert torch.allclose(k_pool.double(), ek, atol=2e-2, rtol=2e-2)
    assert torch.equal(v_pool.double(), ev)
    if dominated is not None:
        assert torch.allclose(out[n - 1, 0].float(), v_pool[dominated[0], 0, dominated[1]].float(), atol=3e-2)


@pytest.mark.parametrize("tcgen05", ["in turn", "together", False])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("d,n_q,n_kv,page_size", [(64, 8, 2, 16), (128, 4, 2, 64), (128, 16, 8, 16)])
@pytest.mark.parametrize("query_len", [64, 300])
def test_prompt_attention_finds_single_keys(kernels, monkeypatch, query_len, d, n_q, n_kv, page_size, window, tcgen05):
    """Prompt portions (the tcgen05 kernel, its softmax groups taking the key tiles in turn or working on each together,
    and the four-warp mma.sync kernel in its place): one key is made to
    dominate one query row, and the output of that row must be that key's value row when the key is visible
    and must not be when the causal mask or the window hides it.  Keys at the places where an index can be
    off by one: key 0, both sides of a 128-key tile edge, a page's last slot, the diagonal, one past the
    diagonal, and both sides of the window's far edge; for the first and the last row of a portion that
    starts in the middle of a page."""
    monkeypatch.setattr(kernels, "USE_TCGEN05_ATTENTION", bool(tcgen05))
    monkeypatch.setattr(kernels, "ATTENTION_IN_TURNS", tcgen05 == "in turn")
    dtype, length = torch.bfloat16, 707
    case = _attention_case(dtype, n_q, n_kv, d, page_size, [length, 90], [query_len, 17], 33)
    q, k_pool, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q, max_ctx = case
    group = n_q // n_kv
    first_pos = length - query_len
    assert first_pos % page_size != 0
    for row in (0, query_len - 1, query_len // 2):
        pos = first_pos + row
        lowest = 0 if window is None else pos - window + 1
        targets = {0, 127, 128, page_size - 1, (pos // page_size) * page_size - 1, pos - 1, pos, pos + 1, 383, 384}
        if window is not None:
            targets |= {lowest - 1, lowest, lowest + 1}
        for target in sorted(t for t in targets if 0 <= t < length):
            visible = lowest <= target <= pos
            kp = k_pool.clone()
            page, offset = int(tables[0, target // page_size]), target % page_size
            for head in (0, n_q - 1):
                kp[page, head // group, offset] = (q[row, head].float() * 40).to(dtype)
            out = torch.empty_like(q)
            kernels.paged_attention(q, kp, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                                    max_ctx, d ** -0.5, window, out)
            kernels.check_device_errors(q.device)
            for head in (0, n_q - 1):
                found = torch.allclose(out[row, head].float(), v_pool[page, head // group, offset].float(), atol=3e-2)
                assert found == visible, (row, target, head, visible)
    # and the whole output, dominant keys and all, against the plain kernel
    _check_attention(kernels, dtype, (q, kp, v_pool, tables, request_of_token, positions, query_start, context_lens, max_q,
                                      max_ctx), d, window)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 331, 72), (37, 384, 96), (64, 64, 16), (65, 130, 200), (130, 257, 1031)])
def test_linear_float32(kernels, m, n, k):
    x, w = rand((m, k), torch.float32, 40), rand((n, k), torch.float32, 41)
    out = torch.empty((m, n), dtype=torch.float32).cuda()
    kernels.linear(x, w, out)
    expected = x.double() @ w.double().T
    assert torch.allclose(out.double(), expected, atol=1e-5 * k ** 0.5, rtol=1e-5)
    # a row's result does not depend on the rows beside it
    alone = torch.empty((1, n), dtype=torch.float32).cuda()
    kernels.linear(x[m // 2:m // 2 + 1].contiguous(), w, alone)
    assert torch.equal(alone[0], out[m // 2])


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 331, 72), (37, 384, 96), (130, 264, 1032)])
def test_linear_bfloat16(kernels, out_dtype, m, n, k):
    x, w = rand((m, k), torch.bfloat16, 42), rand((n, k), torch.bfloat16, 43)
    out = torch.empty((m, n), dtype=out_dtype).cuda()
    kernels.linear(x, w, out)
    expected = x.double() @ w.double().T
    assert torch.allclose(out.double(), expected, atol=2e-2 * k ** 0.5 if out_dtype == torch.bfloat16 else 1e-3, rtol=1e-2)


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 16, 8), (1, 331, 72), (3, 2048, 2048), (8, 500, 1032), (9, 100, 256), (16, 37, 96),
                                   (17, 384, 200), (33, 64, 6144), (64, 331, 264)])
def test_linear_few_rows(kernels, out_dtype, m, n, k):
    """The weight-streaming kernel of decode steps: every row-count class, ragged N and K."""
    x, w = rand((m, k), torch.bfloat16, 44), rand((n, k), torch.bfloat16, 45, 0.1)
    out = torch.empty((m, n), dtype=out_dtype).cuda()
    kernels.linear(x, w, out)
    expected = x.double() @ w.double().T
    bound = 1e-3 if out_dtype == torch.float32 else 2e-2
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)
    alone = torch.empty((1, n), dtype=out_dtype).cuda()
    kernels.linear(x[m // 2:m // 2 + 1].contiguous(), w, alone)
    if m <= kernels.SKINNY_MAX_ROWS:
        assert torch.equal(alone[0], out[m // 2])      # a row does not depend on the rows beside it
    else:
        assert torch.allclose(alone[0].double(), out[m // 2].double(), atol=bound * max(1.0, float(expected.abs().max())))


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 16, 8), (1, 331, 72), (3, 2048, 2048), (8, 4096, 2048), (8, 2048, 6144), (8, 500, 1032),
                                   (9, 100, 256), (16, 12288, 2048), (17, 384, 200), (33, 640, 6144), (64, 331, 264),
                                   (5, 40000, 512), (64, 4096, 2048)])
def test_linear_stream(kernels, out_dtype, m, n, k):
    """The weight-streaming tcgen05 product: one unit, ragged N and K, tiles split over many blocks (summed
    through the workspace), every row-count class; twice, so that the tickets are seen to be left clean."""
    x, w = rand((m, k), torch.bfloat16, 51, 0.5), rand((n, k), torch.bfloat16, 52, 0.1)
    expected = x.double() @ w.double().T
    bound = 1e-3 if out_dtype == torch.float32 else 1.5e-2
    outs = []
    for _ in range(2):
        out = torch.full((m, n), 7.0, dtype=out_dtype).cuda()
        kernels.linear_stream(x, w, out)
        kernels.check_device_errors(x.device)
        assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    alone = torch.empty((1, n), dtype=out_dtype).cuda()
    kernels.linear_stream(x[m // 2:m // 2 + 1].contiguous(), w, alone)
    assert torch.equal(alone[0], outs[0][m // 2])      # a row does not depend on the rows beside it


WIDE_SIZES = [(1, 48, 72), (8, 12288, 2048), (5, 1040, 200), (3, 2064, 4096), (8, 20000, 264), (7, 2048, 6144), (2, 16, 8),
              (8, 24576, 4096), (4, 2064, 12288), (3, 40000, 6408)]


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", WIDE_SIZES)
def test_linear_wide(kernels, out_dtype, m, n, k):
    """The product for weights of many rows: one slot and a ring that wraps many times, one to eight 16-row
    tiles per block, blocks that walk several groups of rows, K walked in parts (activations too large for
    shared memory), ragged N and K."""
    x, w = rand((m, k), torch.bfloat16, 53, 0.5), rand((n, k), torch.bfloat16, 54, 0.1)
    expected = x.double() @ w.double().T
    bound = 1e-3 if out_dtype == torch.float32 else 1.5e-2
    out = torch.full((m, n), 7.0, dtype=out_dtype).cuda()
    kernels.linear_wide(x, w, out)
    kernels.check_device_errors(x.device)
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)
    alone = torch.empty((1, n), dtype=out_dtype).cuda()
    kernels.linear_wide(x[m // 2:m // 2 + 1].contiguous(), w, alone)
    assert torch.equal(alone[0], out[m // 2])            # a row does not depend on the rows beside it


@pytest.mark.parametrize("m,n,k", WIDE_SIZES)
def test_linear_wide_gated(kernels, m, n, k):
    """The same kernel storing silu(gate) * up, against the plain product followed by the plain activation."""
    inter = n // 2 // 8 * 8
    x = rand((m, k), torch.bfloat16, 55, 0.5)
    gate, up = rand((inter, k), torch.bfloat16, 56, 0.1), rand((inter, k), torch.bfloat16, 57, 0.1)
    w = kernels.interleave_gate_up(gate, up)
    assert torch.equal(w[16:24], gate[8:16]) and torch.equal(w[24:32], up[8:16]) if inter >= 16 else True
    out = torch.full((m, inter), 7.0, dtype=torch.bfloat16).cuda()
    kernels.linear_wide(x, w, out, gated=True)
    kernels.check_device_errors(x.device)
    g, u = (x.double() @ gate.double().T).bfloat16().double(), (x.double() @ up.double().T).bfloat16().double()
    expected = g * torch.sigmoid(g) * u
    # the factors are rounded to bfloat16 on both sides; one that falls the other way moves the product by 2^-8
    assert torch.allclose(out.double(), expected, atol=1.5e-2 * max(1.0, float(expected.abs().max())), rtol=1.5e-2)


def test_linear_wide_ring_slots_return_to_the_same_team(kernels):
    """A weight whose blocks take eight tiles has room for five 32 KB slots in its ring and sixteen slots to walk: a
    slot must always come back to the team of warps that had it (a team waits by the parity of the barrier's phase,
    which cannot tell the phase after next from this one), so with an odd ring the teams take the slots by their
    place in it.  Many runs, all with the same bits, against float64."""
    m, n, k = 8, 40960, 2048
    x, w = rand((m, k), torch.bfloat16, 76, 0.5), rand((n, k), torch.bfloat16, 77, 0.1)
    expected = x.double() @ w.double().T
    first = None
    for _ in range(20):
        out = torch.full((m, n), 7.0, dtype=torch.float32).cuda()
        kernels.linear_wide(x, w, out)
        kernels.check_device_errors(x.device)
        if first is None:
            first = out
            assert torch.allclose(out.double(), expected, atol=2e-3 * max(1.0, float(expected.abs().max())), rtol=2e-3)
        else:
            assert torch.equal(out, first)


@pytest.mark.parametrize("m,n,k", [(8, 24576, 4096), (5, 40000, 264)])
def test_linear_wide_blocks_that_walk_many_groups(kernels, monkeypatch, m, n, k):
    """With the switch on, a weight of more rows than one wave of blocks takes is walked by one block per
    multiprocessor, group after group, through one ring (off, it runs as several waves of blocks)."""
    x, w = rand((m, k), torch.bfloat16, 74, 0.5), rand((n, k), torch.bfloat16, 75, 0.1)
    expected = x.double() @ w.double().T
    for switch in ("0", "1"):
        monkeypatch.setenv("MINISERVE_B200_WIDE_MANY", switch)
        out = torch.full((m, n), 7.0, dtype=torch.bfloat16).cuda()
        kernels.linear_wide(x, w, out)
        kernels.check_device_errors(x.device)
        assert torch.allclose(out.double(), expected, atol=1.5e-2 * max(1.0, float(expected.abs().max())), rtol=1.5e-2)
        # a row alone gives the bits it has in the batch: which warps sum which part of K follows from the weight's
        # sizes only (the two forms cut K into slots of different sizes, so they may round differently from each other)
        alone = torch.full((1, n), 7.0, dtype=torch.bfloat16).cuda()
        kernels.linear_wide(x[m - 1:], w, alone)
        assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("norm_dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,k,n_next,gated", [
    (8, 2048, 2048, 4096, False), (1, 2048, 6144, 12288, True), (5, 1040, 200, 528, False), (3, 2064, 4096, 4128, True),
    (8, 72, 64, 48, False), (2, 48, 64, 32, True)])
def test_norm_folded_into_the_products_around_it(kernels, norm_dtype, m, hidden, k, n_next, gated):
    """product -> residual add -> RMSNorm -> product as two kernels: the first adds into the float32 stream, writes
    residual * norm weight and its blocks' sums of squares; the second divides its results by the rows' root mean
    square (before the activation, in its gated form).  Against the four steps in float64; sizes with one to
    eight tiles per block, ragged columns, one to eight rows; and a row alone gives the same bits as in a batch."""
    eps = 1e-5
    x, w = rand((m, k), torch.bfloat16, 80, 0.5), rand((hidden, k), torch.bfloat16, 81, 0.1)
    residual0 = rand((m, hidden), torch.float32, 82, 2.0)
    norm_w = (1 + rand((hidden,), torch.float32, 83, 0.1)).to(norm_dtype)
    w_next = rand((n_next, hidden), torch.bfloat16, 84, 0.05)
    if gated:
        w_next = kernels.interleave_gate_up(w_next[:n_next // 2].contiguous(), w_next[n_next // 2:].contiguous())

    def run(x_rows, residual_rows):
        rows = x_rows.shape[0]
        residual = residual_rows.clone()
        x_next = torch.empty((rows, hidden), dtype=torch.bfloat16).cuda()
        partials = torch.full((kernels.wide_blocks(hidden, k), 8), float("nan"), dtype=torch.float32).cuda()
        stats = kernels.linear_wide_residual(x_rows, w, residual, norm_w, eps, x_next, partials)
        out = torch.empty((rows, n_next // 2 if gated else n_next), dtype=torch.bfloat16).cuda()
        (kernels.gated_up if gated else kernels.linear)(x_next, w_next, out, row_stats=stats)
        kernels.check_device_errors(x.device)
        return residual, x_next, partials, out

    assert kernels.fold_supported(m, torch.bfloat16, w, w_next, gated)
    assert not kernels.fold_supported(9, torch.bfloat16, w, w_next, gated) and not kernels.fold_supported(m, torch.float32, w, w_next, gated)
    residual, x_next, partials, out = run(x, residual0)
    expected_residual = residual0.double() + x.double() @ w.double().T
    assert torch.allclose(residual.double(), expected_residual, atol=1e-4, rtol=1e-5)
    assert torch.allclose(x_next.double(), expected_residual * norm_w.double(), atol=1e-2, rtol=1e-2)
    squares = partials[:kernels.wide_blocks(hidden, k), :m].double().sum(dim=0)
    assert torch.allclose(squares, expected_residual.pow(2).sum(dim=1), rtol=1e-5)
    normed = (expected_residual * torch.rsqrt(expected_residual.pow(2).mean(dim=1, keepdim=True) + eps) * norm_w.double())
    product = normed @ w_next.double().T
    if gated:
        product = product.bfloat16().double()
        inter = n_next // 2
        paired = product.view(m, inter // 8, 2, 8)
        g, u = paired[:, :, 0].reshape(m, inter), paired[:, :, 1].reshape(m, inter)
        product = g * torch.sigmoid(g) * u
    assert torch.allclose(out.double(), product, atol=2e-2 * max(1.0, float(product.abs().max())), rtol=2e-2)
    row = m // 2
    alone = run(x[row:row + 1].contiguous(), residual0[row:row + 1].contiguous())
    assert torch.equal(alone[0][0], residual[row]) and torch.equal(alone[1][0], x_next[row]) and torch.equal(alone[3][0], out[row])


@pytest.mark.parametrize("norm_dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,k,n_next,gated", [
    (2048, 2048, 2048, 4096, False), (2100, 2048, 6144, 12288, True), (300, 1040, 200, 528, False), (257, 520, 136, 544, True),
    (5000, 264, 64, 256, False)])
def test_norm_folded_into_many_row_products(kernels, norm_dtype, m, hidden, k, n_next, gated):
    """The same fold for many rows, in the kernel in which two thread blocks share a tile: the first product adds into
    the float32 stream through shared memory (boxes fetched and stored by TMA), writes residual * norm weight and
    one sum of squares per row and column tile; the second multiplies its results by the rows' factors.  Against
    the four steps in float64; ragged rows and columns, more tiles than pairs of multiprocessors; and a row tile
    alone gives the same bits as among others."""
    eps = 1e-5
    x, w = rand((m, k), torch.bfloat16, 80, 0.5), rand((hidden, k), torch.bfloat16, 81, 0.1)
    residual0 = rand((m, hidden), torch.float32, 82, 2.0)
    norm_w = (1 + rand((hidden,), torch.float32, 83, 0.1)).to(norm_dtype)
    w_next = rand((n_next, hidden), torch.bfloat16, 84, 0.05)
    if gated:
        w_next = kernels.interleave_gate_up(w_next[:n_next // 2].contiguous(), w_next[n_next // 2:].contiguous())

    def run(x_rows, residual_rows):
        rows = x_rows.shape[0]
        residual = residual_rows.clone()
        x_next = torch.full((rows, hidden), 7.0, dtype=torch.bfloat16).cuda()
        partials = torch.full(kernels.residual_partials_shape(rows, hidden, k), float("nan"), dtype=torch.float32).cuda()
        stats = kernels.linear_residual(x_rows, w, residual, norm_w, eps, x_next, partials)
        assert stats.per_row and stats.count == kernels.pair_column_tiles(hidden)
        out = torch.full((rows, n_next // 2 if gated else n_next), 7.0, dtype=torch.bfloat16).cuda()
        (kernels.gated_up if gated else kernels.linear)(x_next, w_next, out, row_stats=stats)
        kernels.check_device_errors(x.device)
        return residual, x_next, partials, out

    residual, x_next, partials, out = run(x, residual0)
    expected_residual = residual0.double() + x.double() @ w.double().T
    assert torch.allclose(residual.double(), expected_residual, atol=1e-4, rtol=1e-5)
    assert torch.allclose(x_next.double(), expected_residual * norm_w.double(), atol=1e-2, rtol=1e-2)
    # (the sums are those of the stream as the kernel holds it, in float32)
    squares = partials.double().sum(dim=0)
    assert torch.allclose(squares, residual.double().pow(2).sum(dim=1), rtol=1e-5)
    normed = (expected_residual * torch.rsqrt(expected_residual.pow(2).mean(dim=1, keepdim=True) + eps) * norm_w.double())
    product = normed @ w_next.double().T
    if gated:
        product = product.bfloat16().double()
        inter = n_next // 2
        paired = product.view(m, inter // 8, 2, 8)
        g, u = paired[:, :, 0].reshape(m, inter), paired[:, :, 1].reshape(m, inter)
        product = g * torch.sigmoid(g) * u
    assert torch.allclose(out.double(), product, atol=2e-2 * max(1.0, float(product.abs().max())), rtol=2e-2)
    first = min(256, m) - 9
    alone = run(x[first:first + 9].contiguous(), residual0[first:first + 9].contiguous())
    assert torch.equal(alone[0], residual[first:first + 9]) and torch.equal(alone[1], x_next[first:first + 9])
    assert torch.equal(alone[3], out[first:first + 9])


@pytest.mark.parametrize("m,k,n_q,n_kv,norm,rotate,page_size,folded", [
    (2048, 2048, 16, 8, True, True, 64, False), (300, 136, 3, 1, True, True, 16, False), (1000, 256, 4, 2, False, True, 8, False),
    (520, 512, 2, 2, True, False, 32, False), (2100, 2048, 16, 8, True, True, 64, True), (257, 64, 5, 1, True, True, 4, True)])
def test_qkv_projection_with_norm_rotation_and_append_in_its_epilogue(kernels, m, k, n_q, n_kv, norm, rotate, page_size, folded):
    """The q/k/v projection whose tiles are normed, rotated and appended as they leave the tensor cores, against the
    same product followed by the separate norm + rotation + append kernel: the same roundings in the same places,
    so q and both pools agree to a bfloat16 rounding step (the sums of squares are added in another order); head
    counts that leave a tile half empty or straddle q, k and v inside a tile, ragged rows, rows that are not stored,
    scattered slots, and a norm folded in before."""
    d = 128
    heads = n_q + 2 * n_kv
    x, w = rand((m, k), torch.bfloat16, 90, 0.5), rand((heads * d, k), torch.bfloat16, 91, 0.2)
    q_w = (1 + rand((d,), torch.float32, 92, 0.2)).to(torch.bfloat16) if norm else None
    k_w = (1 + rand((d,), torch.float32, 93, 0.2)).to(torch.bfloat16) if norm else None
    cos_sin = None
    if rotate:
        angles = torch.rand((m, d // 2), generator=torch.Generator().manual_seed(94)) * 6.28
        cos_sin = torch.stack((torch.cos(angles), torch.sin(angles)), dim=-1).float().cuda().contiguous()
    pages = (m + page_size - 1) // page_size + 3
    order = torch.randperm(pages * page_size, generator=torch.Generator().manual_seed(95))[:m].to(torch.int32)
    order[5] = -1                                           # a row that is computed but not stored
    slots = order.cuda()
    stats = None
    if folded:
        partials = (rand((3, m), torch.float32, 96).abs() * k / 3).contiguous()
        stats = kernels.RowStats(partials, 3, 1e-6, per_row=True)

    def pools():
        return [torch.full((pages, n_kv, page_size, d), 3.0, dtype=torch.bfloat16).cuda() for _ in range(2)]

    k_ref, v_ref = pools()
    qkv = torch.empty((m, heads * d), dtype=torch.bfloat16).cuda()
    kernels.linear_pair(x, w, qkv, row_stats=stats)
    q_ref = torch.empty((m, n_q, d), dtype=torch.bfloat16).cuda()
    kernels.qk_norm_rope_append(qkv, slots, q_w, k_w, 1e-6, cos_sin, d, False, k_ref, v_ref, n_q, n_kv, d, q_ref)
    k_pool, v_pool = pools()
    q = torch.full((m, n_q, d), 7.0, dtype=torch.bfloat16).cuda()
    kernels.linear_pair_qkv(x, w, slots, q_w, k_w, 1e-6, cos_sin, k_pool, v_pool, n_q, n_kv, q, row_stats=stats)
    kernels.check_device_errors(x.device)
    assert torch.equal(v_pool, v_ref)                       # values are only rounded and stored
    for got, expected in ((q, q_ref), (k_pool, k_ref)):
        scale = float(expected.float().abs().max())
        assert torch.allclose(got.float(), expected.float(), atol=scale * 2 ** -8, rtol=2 ** -7)
        assert float((got != expected).float().mean()) < 0.02          # and nearly all of them exactly


def test_many_row_products_choose_between_the_own_kernel_and_the_library_by_measurement(kernels, monkeypatch):
    """Every kind of many-row product is timed both ways once per count of row tiles and weight shape, the faster way
    is kept with the times, and a second question measures nothing."""
    monkeypatch.setattr(kernels, "LINEAR_TUNING", True)
    monkeypatch.setattr(kernels, "_many_row_choices", {})
    n_q, n_kv = 4, 2
    weights = {"plain": rand((1024, 512), torch.bfloat16, 1, 0.1), "gated": rand((2048, 512), torch.bfloat16, 2, 0.1),
               "add": rand((512, 1024), torch.bfloat16, 3, 0.1), "qkv": rand(((n_q + 2 * n_kv) * 128, 512), torch.bfloat16, 4, 0.1)}
    first = {kind: kernels._pair_or_library(kind, 600, weight, n_q, n_kv) for kind, weight in weights.items()}
    kernels.check_device_errors(torch.device("cuda"))
    assert set(first.values()) <= {"pair", "wide", "library"}
    recorded = kernels.many_row_choices()
    for kind, weight in weights.items():
        choice, times = recorded[(0, kind, 3, weight.shape[0], weight.shape[1])]
        assert choice == first[kind] == min(times, key=times.get)
        assert set(times) == ({"pair", "library"} if kind == "qkv" else {"pair", "wide", "library"})
        assert all(0 < t < 1000 for t in times.values())

    def never(*args):
        raise AssertionError("measured twice")

    monkeypatch.setattr(kernels, "_measure_many_rows", never)
    assert {kind: kernels._pair_or_library(kind, 700, weight, n_q, n_kv) for kind, weight in weights.items()} == first
    monkeypatch.setattr(kernels, "LINEAR_TUNING", False)
    assert kernels._pair_or_library("plain", 5000, weights["plain"]) == "pair"        # no measurement: the own kernel


def test_many_row_fold_is_offered_where_it_pays(kernels, monkeypatch):
    monkeypatch.setattr(kernels, "LINEAR_TUNING", False)        # the rule alone
    hidden, inter = 2048, 6144
    o, gate_up = rand((hidden, hidden), torch.bfloat16, 1), rand((2 * inter, hidden), torch.bfloat16, 2)
    assert kernels.fold_supported(4096, torch.bfloat16, o, gate_up, True)
    assert not kernels.fold_supported(2048, torch.bfloat16, o, gate_up, True)      # one tile per pair: nothing to overlap with
    assert not kernels.fold_supported(3072, torch.bfloat16, o, gate_up, True)      # 96 tiles of o on 74 pairs
    assert not kernels.fold_supported(4096, torch.float32, o, gate_up, True)
    assert not kernels.fold_supported(64, torch.bfloat16, o, gate_up, True)


def test_linear_wide_refusals(kernels):
    x, w = rand((9, 64), torch.bfloat16, 58), rand((32, 64), torch.bfloat16, 59)
    with pytest.raises(kernels.KernelError, match="at most 8"):
        kernels.linear_wide(x, w, torch.empty((9, 32), dtype=torch.bfloat16).cuda())
    with pytest.raises(kernels.KernelError, match="multiple of 8"):
        kernels.linear_wide(rand((2, 60), torch.bfloat16, 58), rand((32, 60), torch.bfloat16, 59),
                            torch.empty((2, 32), dtype=torch.bfloat16).cuda())
    with pytest.raises(kernels.KernelError, match="multiple of 16"):
        kernels.linear_wide(x[:2].contiguous(), w[:24].contiguous(), torch.empty((2, 12), dtype=torch.bfloat16).cuda(), gated=True)
    assert kernels.wide_supports(64, 12) == 0               # an inner size that is no multiple of 8
    assert kernels.wide_supports(4096, 2048) == 2           # one group of rows per block, the activations whole in shared memory
    assert kernels.wide_supports(4096, 12288) in (0, 1)     # K in parts: taken, but offered to the choice only on request
    assert kernels.wide_supports(151936, 2048) in (0, 1)    # several groups of rows per block: the same


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,inter,k", [(1, 200, 72), (8, 6144, 2048), (20, 224, 96), (3, 8, 64)])
def test_gated_up(kernels, dtype, m, inter, k):
    """What the feed-forward part calls: whichever way the kernels choose, the plain result."""
    x = rand((m, k), dtype, 60, 0.5)
    w = kernels.interleave_gate_up(rand((inter, k), dtype, 61, 0.1), rand((inter, k), dtype, 62, 0.1))
    out = torch.empty((m, inter), dtype=dtype).cuda()
    kernels.gated_up(x, w, out)
    kernels.check_device_errors(x.device)
    expected = torch.empty((m, inter), dtype=torch.float64).cuda()
    plain_ops.gated_up(x, w, expected)
    bound = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,inter", [(1, 72, 200), (8, 2048, 6144), (20, 96, 224), (64, 331, 128), (100, 96, 224), (5, 64, 100)])
def test_gated_linear(kernels, dtype, m, n, inter):
    gate_up, w = rand((m, 2 * inter), dtype, 46, 2.0), rand((n, inter), dtype, 47, 0.1)
    out = torch.empty((m, n), dtype=dtype).cuda()
    kernels.gated_linear(gate_up, w, out)
    expected = torch.empty((m, n), dtype=torch.float64).cuda()
    plain_ops.gated_linear(gate_up, w, expected)
    bound = 1e-4 if dtype == torch.float32 else 2e-2
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)


@pytest.mark.parametrize("m,n,k,out_dtype,add", [
    (128, 128, 64, torch.bfloat16, False), (130, 264, 72, torch.bfloat16, False), (1, 40, 8, torch.float32, False),
    (300, 331, 200, torch.float32, False), (2048, 2048, 2048, torch.bfloat16, False), (257, 6144, 2048, torch.bfloat16, False),
    (512, 2048, 6144, torch.float32, True), (150, 96, 224, torch.float32, True)])
def test_linear_tcgen05(kernels, m, n, k, out_dtype, add):
    """The TMA + tcgen05 + tensor-memory product: whole and ragged tiles, both epilogues, no wait given up."""
    x, w = rand((m, k), torch.bfloat16, 48, 0.5), rand((n, k), torch.bfloat16, 49, 0.1)
    expected = x.double() @ w.double().T
    if add:
        out = rand((m, n), torch.float32, 50)
        expected = expected + out.double()
    else:
        out = torch.full((m, n), 7.0, dtype=out_dtype).cuda()
    kernels.linear_tcgen05(x, w, out, add=add)
    kernels.check_device_errors(x.device)
    bound = 1e-3 if out_dtype == torch.float32 else 1.5e-2
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)


@pytest.mark.parametrize("m,n,k,out_dtype,mode", [
    (256, 256, 64, torch.bfloat16, "store"), (130, 264, 72, torch.bfloat16, "store"), (1, 40, 8, torch.float32, "store"),
    (300, 331, 200, torch.float32, "store"), (2048, 4096, 2048, torch.bfloat16, "store"), (257, 6144, 520, torch.bfloat16, "store"),
    (5000, 2048, 256, torch.bfloat16, "store"), (512, 2048, 6144, torch.float32, "add"), (150, 96, 224, torch.float32, "add"),
    (2048, 12288, 2048, torch.bfloat16, "gated"), (300, 656, 136, torch.bfloat16, "gated"), (40, 16, 64, torch.bfloat16, "gated")])
@pytest.mark.parametrize("wide", [False, True])
def test_linear_pair(kernels, m, n, k, out_dtype, mode, wide):
    """The product in which two thread blocks share a 256 x 256 tile (tcgen05 with cta_group::2): whole and ragged
    tiles, more tiles than pairs of multiprocessors, every epilogue, no wait given up."""
    x, w = rand((m, k), torch.bfloat16, 48, 0.5), rand((n, k), torch.bfloat16, 49, 0.1)
    expected = x.double() @ w.double().T
    if mode == "add":
        out = rand((m, n), torch.float32, 50)
        expected = expected + out.double()
    elif mode == "gated":
        out = torch.full((m, n // 2), 7.0, dtype=out_dtype).cuda()
        blocks = expected.view(m, n // 16, 2, 8)
        expected = (torch.nn.functional.silu(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(m, n // 2)
    else:
        out = torch.full((m, n), 7.0, dtype=out_dtype).cuda()
    kernels.linear_pair(x, w, out, add=mode == "add", gated=mode == "gated", wide=wide)     # wide: tiles of 256 x 512
    kernels.check_device_errors(x.device)
    bound = 1e-3 if out_dtype == torch.float32 else 1.5e-2
    assert torch.allclose(out.double(), expected, atol=bound * max(1.0, float(expected.abs().max())), rtol=bound)


def records_tensor(rows):
    words = [struct.unpack("<8i", struct.pack("<ffiIIiii", t, p, k, seed & 0xFFFFFFFF, seed >> 32, 0, 0, 0))
             for (t, p, k, seed) in rows]
    return torch.tensor(words, dtype=torch.int32).cuda()


@pytest.mark.parametrize("vocab", [1, 7, 331, 5000, 151936])
def test_argmax_lowest_index_on_ties(kernels, vocab):
    logits = rand((3, vocab), torch.float32, 50)
    if vocab > 5:
        logits[1, 4] = logits[1, vocab - 1] = 99.0
    out = torch.empty(3, dtype=torch.int32).cuda()
    kernels.sample(logits, None, None, None, out)
    expected = [int(torch.argmax(row)) for row in logits.cpu()]
    if vocab > 5:
        expected[1] = 4
    assert out.tolist() == expected


@pytest.mark.parametrize("vocab", [13, 331, 4099])
def test_sample_matches_plain_rule(kernels, vocab):
    rows = [(0.0, 1.0, 0, 1), (0.8, 1.0, 0, 2), (1.0, 1.0, 5, 3), (0.7, 0.9, 0, 2 ** 40 + 5), (1.3, 0.5, 11, 7),
            (2.0, 0.3, 3, 9), (1.0, 1.0, 1, 4), (0.5, 0.999, vocab, 5)]
    records = records_tensor(rows)
    logits = rand((len(rows), vocab), torch.float32, 60, 2.0)
    slot_of_row = torch.arange(len(rows), dtype=torch.int32).cuda()
    for draw in (0, 1, 17):
        draw_index = torch.full((len(rows),), draw, dtype=torch.int32).cuda()
        out = torch.empty(len(rows), dtype=torch.int32).cuda()
        kernels.sample(logits, records, slot_of_row, draw_index, out)
        for r, (t, p, k, seed) in enumerate(rows):
            expected = plain.plain_sample(logits[r].cpu(), t, k, p, seed, draw)
            assert int(out[r]) == expected, (r, draw)


def test_sample_keeps_exactly_k_under_ties(kernels):
    vocab = 50
    logits = torch.zeros((1, vocab), dtype=torch.float32)
    logits[0, [3, 9, 20, 31]] = 5.0          # four equal maxima, top_k = 2 keeps indices 3 and 9
    records = records_tensor([(1.0, 1.0, 2, 11)])
    seen = set()
    for draw in range(64):
        out = torch.empty(1, dtype=torch.int32).cuda()
        kernels.sample(logits.cuda(), records, torch.zeros(1, dtype=torch.int32).cuda(),
                       torch.tensor([draw], dtype=torch.int32).cuda(), out)
        seen.add(int(out[0]))
    assert seen == {3, 9}


def test_sample_follows_the_softmax(kernels):
    """Frequencies over many draws approach the softmax of logits / temperature."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]], dtype=torch.float32).cuda()
    records = records_tensor([(0.7, 1.0, 0, 123)])
    draws = 4000
    big = logits.expand(draws, -1).contiguous()
    out = torch.empty(draws, dtype=torch.int32).cuda()
    kernels.sample(big, records, torch.zeros(draws, dtype=torch.int32).cuda(),
                   torch.arange(draws, dtype=torch.int32).cuda(), out)
    freq = torch.bincount(out.long().cpu(), minlength=5).double() / draws
    expected = torch.softmax(logits[0].double().cpu() / 0.7, dim=0)
    assert float((freq - expected).abs().max()) < 0.03
