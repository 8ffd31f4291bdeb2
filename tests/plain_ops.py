"""Plain PyTorch statements of what each kernel entry point computes.

Two uses: the GPU tests compare every kernel alone with the function of the same name here
(computed in float64 from the same inputs), and the CPU tests put these functions in the
kernels' place (``install``) so that the host-side logic of the engine (batching, cache
manager, step function) can be exercised on a machine without a GPU.  Nothing here is used by
the package itself.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

import plain_qwen3 as plain


def scale_softcap(x, scale=1.0, cap=None):
    x.mul_(scale)
    if cap:
        x.copy_(cap * torch.tanh(x / cap))


def embedding(tokens, table, out, scale=1.0):
    out.copy_((scale * table[tokens.long()].double()).to(out.dtype))


def add_rmsnorm(residual, delta, weight, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            residual += delta.to(residual.dtype)
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].to(residual.dtype)
    x = x.double()
    y = weight.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(y.to(out.dtype))


def rmsnorm(x, weight, eps, out):
    xd = x.double()
    y = weight.double() * (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(y.to(out.dtype))


def rope_table(positions, inv_freq, cos_sin):
    angles = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).double()
    cos_sin[..., 0] = angles.cos().to(cos_sin.dtype)
    cos_sin[..., 1] = angles.sin().to(cos_sin.dtype)


def rotate(x, cos_sin, rotary_dim, interleaved):
    """x [N, heads, d] float64; cos_sin [N, rotary_dim/2, 2]."""
    cos, sin = cos_sin[..., 0].double()[:, None, :], cos_sin[..., 1].double()[:, None, :]
    out = x.clone()
    half = rotary_dim // 2
    if interleaved:
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2] = a * cos - b * sin
        out[..., 1:rotary_dim:2] = b * cos + a * sin
    else:
        a, b = x[..., :half], x[..., half:rotary_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rotary_dim] = b * cos + a * sin
    return out


def qk_norm_rope_append(qkv, slots, q_weight, k_weight, eps, cos_sin, rotary_dim, interleaved, k_pool, v_pool,
                        n_q, n_kv, head_dim, q_out):
    n = qkv.shape[0]
    heads = qkv.view(n, n_q + 2 * n_kv, head_dim).double()
    q, k, v = heads[:, :n_q], heads[:, n_q:n_q + n_kv], heads[:, n_q + n_kv:]

    def norm(x, w):
        if w is None:
            return x
        return w.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))

    q, k = norm(q, q_weight), norm(k, k_weight)
    if cos_sin is not None:
        q, k = rotate(q, cos_sin, rotary_dim, interleaved), rotate(k, cos_sin, rotary_dim, interleaved)
    q_out.copy_(q.to(q_out.dtype))
    page_size = k_pool.shape[2]
    for token in range(n):
        slot = int(slots[token])
        if slot < 0:
            continue
        page, offset = divmod(slot, page_size)
        k_pool[page, :, offset, :] = k[token].to(k_pool.dtype)
        v_pool[page, :, offset, :] = v[token].to(v_pool.dtype)


def silu_mul(gate_up, out, paired=False):
    n, inter = out.shape
    if paired:      # blocks of sixteen columns: eight of the gate, then the same eight of the up projection
        blocks = gate_up.reshape(n, inter // 8, 2, 8)
        g, u = blocks[:, :, 0].reshape(n, inter).double(), blocks[:, :, 1].reshape(n, inter).double()
    else:
        g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def _row_factor(row_stats, size):
    """1 / rms of every row from the partial sums of squares that a folded norm left (kernels.RowStats)."""
    total = row_stats.partials[:row_stats.count].double().sum(dim=0)
    return 1.0 / torch.sqrt(total / size + row_stats.eps)


def gated_up(x, weight, out, row_stats=None):
    gate_up = x.double() @ weight.double().T
    if row_stats is not None:
        gate_up = gate_up * _row_factor(row_stats, x.shape[1])[:x.shape[0], None]
    silu_mul(gate_up.to(x.dtype), out, paired=True)


FOLD_BLOCKS = 3     # the plain stand-in leaves its sums of squares in this many rows, as a kernel of three blocks would


def linear_residual(x, weight, residual, norm_weight, eps, x_next, partials):
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    residual += (x.double() @ weight.double().T).to(residual.dtype)
    x_next.copy_((residual.double() * norm_weight.double()).to(x_next.dtype))
    partials.zero_()
    for block, columns in enumerate(torch.arange(residual.shape[1]).chunk(FOLD_BLOCKS)):
        partials[block, :residual.shape[0]] = residual[:, columns].double().pow(2).sum(dim=1).to(partials.dtype)
    return kernels.RowStats(partials, FOLD_BLOCKS, eps, per_row=partials.shape[1] != 8)


def linear_add(x, weight, residual):
    residual += (x.double() @ weight.double().T).to(residual.dtype)


def paged_attention(q, k_pool, v_pool, block_tables, request_of_token, positions, query_start, context_lens,
                    max_query_len, max_context_len, scale, window, out, host_query_start=None, softcap=None,
                    bias_slopes=None):
    n, n_q, d = q.shape
    n_kv, page_size = k_pool.shape[1], k_pool.shape[2]
    group = n_q // n_kv
    for token in range(n):
        pos = int(positions[token])
        table = block_tables[int(request_of_token[token])]
        first = max(0, pos - window + 1) if window else 0
        keys = torch.arange(first, pos + 1)
        pages = table[(keys // page_size).long()].long()
        offsets = (keys % page_size).long()
        k = k_pool[pages, :, offsets, :].double()      # [keys, n_kv, d]
        v = v_pool[pages, :, offsets, :].double()
        for head in range(n_q):
            scores = (k[:, head // group, :] @ q[token, head].double()) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if bias_slopes is not None:
                scores = scores + float(bias_slopes[head]) * (keys - pos).double()
            p = torch.softmax(scores, dim=0)
            out[token, head] = (p @ v[:, head // group, :]).to(out.dtype)


def linear(x, weight, out, row_stats=None):
    product = x.double() @ weight.double().T
    if row_stats is not None:
        product = product * _row_factor(row_stats, x.shape[1])[:x.shape[0], None]
    out.copy_(product.to(out.dtype))


def gated_linear(gate_up, weight, out):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    hidden = (g * torch.sigmoid(g) * u).to(gate_up.dtype)
    out.copy_((hidden.double() @ weight.double().T).to(out.dtype))


def sample(logits, records, slot_of_row, draw_index, out):
    import struct

    for row in range(logits.shape[0]):
        if records is None:
            out[row] = int(torch.argmax(logits[row]))
            continue
        words = records[int(slot_of_row[row])].tolist()
        temperature, top_p, top_k, seed_lo, seed_hi, *_ = struct.unpack("<ffiIIiii", struct.pack("<8i", *words))
        out[row] = plain.plain_sample(logits[row].cpu(), temperature, top_k, top_p, seed_lo | (seed_hi << 32),
                                      int(draw_index[row]))


def install(monkeypatch) -> None:
    """Puts the functions above in place of the kernel bindings (CPU tests of host logic only)."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    for name in ("embedding", "add_rmsnorm", "rmsnorm", "rope_table", "qk_norm_rope_append", "silu_mul",
                 "paged_attention", "linear", "gated_linear", "gated_up", "sample", "scale_softcap"):
        monkeypatch.setattr(kernels, name, globals()[name])
    monkeypatch.setattr(kernels, "attention_kernels", lambda *sizes: {"decode": "plain", "prompt": "plain"})
    # norms folded into the products around them: offered for steps of up to eight rows and for steps of many
    # (here: 24 and more), as on the device, with the two layouts of the sums of squares
    monkeypatch.setattr(kernels, "linear_residual", linear_residual)
    monkeypatch.setattr(kernels, "residual_partials_shape", lambda rows, n, k: (FOLD_BLOCKS, 8 if rows <= 8 else rows))
    monkeypatch.setattr(kernels, "fold_supported", lambda rows, dtype, producer, consumer, gated=False: 0 < rows <= 8 or rows >= 24)
    monkeypatch.setattr(kernels, "qkv_in_product_supported", lambda *sizes: False)
    # products that add into the residual stream themselves: offered for steps of 12 to 23 rows
    monkeypatch.setattr(kernels, "linear_add", linear_add)
    monkeypatch.setattr(kernels, "add_in_product_supported", lambda rows, dtype, weight: 12 <= rows < 24)
