"""Plain torch statements of what each CUDA kernel computes, with the signatures
of ``kairyu_b200.kernels``.  The GPU tests compare every kernel with these; the
CPU tests install them in place of the kernels (``install``) to exercise the
cache, the step function, the scheduler and the replay program without a GPU.
They are test code: the package itself has no implementation but its kernels.
"""

from __future__ import annotations



import torch

import plain_model

DECODE_SPLIT = 128


def embedding(table, ids, out, flag=None):
    out.copy_(table[ids.long()].float())


def patch_tokens(ids, source, sampled, flag=None):
    for t in range(ids.numel()):
        if int(source[t]) >= 0:
            ids[t] = sampled[int(source[t])]


def rmsnorm(x, weight, eps, out, *, delta=None, rows=None):
    if rows is not None:
        v = x[rows.long()].float()
        if delta is not None:
            v = v + delta[rows.long()].float()
    else:
        if delta is not None:
            x.copy_((x.float() + delta.float()).to(x.dtype))
        v = x.float()
    normed = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    out[: normed.shape[0]].copy_(normed.to(out.dtype))


def swiglu(gate_up, out):
    inter = gate_up.shape[1] // 2
    g = gate_up[:, :inter].float()
    u = gate_up[:, inter:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def gather_rows(src, rows, out):
    out.copy_(src[rows.long()])


def qk_norm_rope_kv_write(
    qkv, num_q_heads, num_kv_heads, head_dim, *, positions, row_ids, q_norm_weight=None, k_norm_weight=None,
    eps=0.0, cos=None, sin=None, block_table=None, write_from=None, k_cache=None, v_cache=None, flag=None,
):
    T = qkv.shape[0]
    q_size = num_q_heads * head_dim
    kv_size = num_kv_heads * head_dim
    q = qkv[:, :q_size].float().clone().view(T, num_q_heads, head_dim)
    k = qkv[:, q_size : q_size + kv_size].float().clone().view(T, num_kv_heads, head_dim)
    v = qkv[:, q_size + kv_size :].view(T, num_kv_heads, head_dim)
    if q_norm_weight is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_norm_weight.float()
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_norm_weight.float()
    if cos is not None:
        half = cos.shape[1]
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :]

        def rotate(u):
            a, b, rest = u[..., :half], u[..., half : 2 * half], u[..., 2 * half :]
            return torch.cat((a * c - b * s, b * c + a * s, rest), dim=-1)

        q, k = rotate(q), rotate(k)
    qkv[:, :q_size].copy_(q.reshape(T, q_size).to(qkv.dtype))
    qkv[:, q_size : q_size + kv_size].copy_(k.reshape(T, kv_size).to(qkv.dtype))
    if k_cache is not None:
        page_size = k_cache.shape[1]
        kf = k_cache.view(-1, num_kv_heads, head_dim)
        vf = v_cache.view(-1, num_kv_heads, head_dim)
        for t in range(T):
            pos = int(positions[t])
            row = int(row_ids[t])
            if pos < int(write_from[row]):
                continue
            page = int(block_table[row, pos // page_size])
            assert page >= 0, "write through an absent page"
            slot = page * page_size + pos % page_size
            kf[slot] = k[t].to(k_cache.dtype)
            vf[slot] = v[t]


def _attend_token(q_t, k_cache, v_cache, table, pos, num_q_heads, scale, window):
    """q_t: [Hq, D] fp32 -> [Hq, D] fp32 over keys max(0,pos+1-window)..pos of one request."""
    num_pages, page_size, kv_heads, dim = k_cache.shape
    start = max(0, pos + 1 - window) if window > 0 else 0
    keys = torch.arange(start, pos + 1)
    pages = table[(keys // page_size).long()].long()
    assert (pages >= 0).all(), "read through an absent page"
    slots = pages * page_size + keys % page_size
    k = k_cache.view(-1, kv_heads, dim)[slots].float()
    v = v_cache.view(-1, kv_heads, dim)[slots].float()
    group = num_q_heads // kv_heads
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("hd,khd->hk", q_t, k) * scale
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hk,khd->hd", probs, v)


def paged_attention_generic(q, out, k_cache, v_cache, *, positions, row_ids, block_table, num_q_heads, scale, window=0, flag=None):
    dim = k_cache.shape[-1]
    for t in range(q.shape[0]):
        q_t = q[t, : num_q_heads * dim].float().view(num_q_heads, dim)
        res = _attend_token(q_t, k_cache, v_cache, block_table[int(row_ids[t])], int(positions[t]), num_q_heads, scale, window)
        out[t].copy_(res.reshape(-1).to(out.dtype))


def attention_mma_supported(head_dim, num_q_heads, num_kv_heads):
    return head_dim % 16 == 0 and 16 <= head_dim <= 256 and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 16


def attention_prefill_tile_rows(head_dim):
    return 128 if head_dim <= 128 else 64


def attention_prefill_mma(q, out, k_cache, v_cache, *, qo_indptr, seq_lens, block_table, tile_rows, tile_starts, num_tiles, num_q_heads, scale, window=0, flag=None):
    dim = k_cache.shape[-1]
    for tile in range(num_tiles):
        row = int(tile_rows[tile])
        q0 = int(tile_starts[tile])
        tok0 = int(qo_indptr[row])
        chunk = int(qo_indptr[row + 1]) - tok0
        chunk_pos = int(seq_lens[row]) - chunk
        for i in range(q0, min(q0 + attention_prefill_tile_rows(dim), chunk)):
            t = tok0 + i
            q_t = q[t, : num_q_heads * dim].float().view(num_q_heads, dim)
            res = _attend_token(q_t, k_cache, v_cache, block_table[row], chunk_pos + i, num_q_heads, scale, window)
            out[t].copy_(res.reshape(-1).to(out.dtype))


def attention_decode_mma(q, out, k_cache, v_cache, *, seq_lens, block_table, decode_rows, decode_tokens, num_rows, max_seq_len, num_q_heads, scale, window=0, workspace=None, flag=None, num_splits=None):
    dim = k_cache.shape[-1]
    for slot in range(num_rows):
        row = int(decode_rows[slot])
        t = int(decode_tokens[slot])
        assert int(seq_lens[row]) <= max_seq_len
        q_t = q[t, : num_q_heads * dim].float().view(num_q_heads, dim)
        res = _attend_token(q_t, k_cache, v_cache, block_table[row], int(seq_lens[row]) - 1, num_q_heads, scale, window)
        out[t].copy_(res.reshape(-1).to(out.dtype))


def linear(x, weight, bias, out):
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    out.copy_(y.to(out.dtype))


def linear_swiglu(x, weight_gate_up, out, scratch):
    inter = weight_gate_up.shape[0] // 2
    y = x.float() @ weight_gate_up.float().t()
    g, u = y[:, :inter], y[:, inter:]
    if x.dtype != torch.float32:  # the two-kernel path rounds the product before the gate
        g, u = g.to(x.dtype).float(), u.to(x.dtype).float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def fused_norm_available():
    return False  # the CPU statements keep the norm a step of its own


def argmax(logits, out):
    out.copy_(logits.argmax(dim=-1).to(torch.int32))


def edit_logits(logits, rows, tokens, mul, sub, mask):
    for e in range(rows.numel()):
        r, t = int(rows[e]), int(tokens[e])
        if int(mask[e]):
            logits[r, t] = float("-inf")
            continue
        value = logits[r, t]
        m = float(mul[e])
        if m != 1.0:
            value = value / m if value > 0 else value * m
        logits[r, t] = value - float(sub[e])


def sample_work_floats(rows, vocab):
    return rows * vocab


def sample(logits, work, temperature, top_k, top_p, min_p, seeds, out):
    """Row-wise: the reference's filters and Gumbel-max draw.  ``seeds`` already
    carry the position (mix_seed on the host)."""
    for r in range(logits.shape[0]):
        T = float(temperature[r])
        if T == 0.0:
            out[r] = int(logits[r].argmax())
            continue
        probs = plain_model.filtered_probs(logits[r], T, int(top_k[r]), float(top_p[r]), float(min_p[r]))
        noise = plain_model.gumbel_noise(probs.numel(), int(seeds[r]) & ((1 << 64) - 1))
        out[r] = int(torch.argmax(torch.log(probs).to(torch.float64) + noise))


def logprob_report(logits, rows, tokens, k, values, indices, *, tokens_by_row):
    for r in range(rows.numel()):
        row = int(rows[r])
        logp = torch.log_softmax(logits[row].to(torch.float32), dim=-1)
        token = int(tokens[row] if tokens_by_row else tokens[r])
        values[r, 0] = logp[token]
        if k:
            # largest first, ties by the lower index: sort on (-value, index)
            order = sorted(range(logp.numel()), key=lambda i: (-float(logp[i]), i))[:k]
            for place, index in enumerate(order):
                values[r, 1 + place] = logp[index]
                indices[r, place] = index
            for place in range(len(order), k):
                values[r, 1 + place] = float("-inf")
                indices[r, place] = -1


def linear_rope_ok(*args, **kwargs):
    return False  # the CPU statements keep the product and the rotation apart


_NAMES = [
    "embedding", "patch_tokens", "fused_norm_available", "rmsnorm", "swiglu", "gather_rows", "qk_norm_rope_kv_write", "paged_attention_generic",
    "attention_mma_supported", "attention_prefill_tile_rows", "attention_prefill_mma", "attention_decode_mma", "linear", "linear_swiglu", "argmax",
    "edit_logits", "sample", "sample_work_floats", "logprob_report", "linear_rope_ok",
]


def install(monkeypatch) -> None:
    """Replace the kernels by these functions for one test (CPU runs)."""
    import kairyu_b200.kernels as kernels

    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
