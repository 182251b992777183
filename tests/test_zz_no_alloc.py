"""The decode-attention entry point that allocates nothing
(``kb_attention_decode_mma_static``, csrc/attention_decode_static.h), called
through its exported C symbol the way a C host would, and compared with the
ordinary entry point and with attention written out in fp32 torch, on two calls
in a row.

The entry point is for callers that cannot allocate device memory around the
call (all memory already given to a pool of their own, no allocator of the
process within reach, no torch in the process): the library keeps the scratch
for the per-split partial results itself.  This file sorts last on purpose, so
a run that stops at the first failure has already run everything else.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_BAD_ARG = -1
ERR_SCRATCH_TOO_SMALL = -4
BF16_TOLERANCE = 2e-2  # the bound the other bf16 attention tests use


def _case(seq_lens, Hq, Hkv, D, page_size, seed):
    g = torch.Generator().manual_seed(seed)
    rows = len(seq_lens)
    max_pages = max(-(-s // page_size) for s in seq_lens)
    num_pages = rows * max_pages + 1
    table = (torch.randperm(num_pages - 1, generator=g)[: rows * max_pages] + 1).view(rows, max_pages).to(torch.int32)
    k = (torch.randn(num_pages, page_size, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
    v = torch.randn(num_pages, page_size, Hkv, D, generator=g).to(torch.bfloat16)
    q = (torch.randn(rows, (Hq + 2 * Hkv) * D, generator=g) * 0.5).to(torch.bfloat16)
    dev = lambda t: t.to("cuda")
    return dict(
        q=dev(q), k=dev(k), v=dev(v), table=dev(table), seq_lens=dev(torch.tensor(seq_lens, dtype=torch.int32)),
        rows=dev(torch.arange(rows, dtype=torch.int32)), tokens=dev(torch.arange(rows, dtype=torch.int32)),
        Hq=Hq, Hkv=Hkv, D=D, page_size=page_size, num_pages=num_pages, max_seq_len=max(seq_lens), count=rows,
    )


def _plain_attention(case):
    """softmax(q k^T / sqrt(D)) v per row and head over the row's pages, in fp32 torch."""
    Hq, Hkv, D, page_size = case["Hq"], case["Hkv"], case["D"], case["page_size"]
    group = Hq // Hkv
    out = torch.zeros(case["count"], Hq * D)
    k_all, v_all, table = case["k"].float().cpu(), case["v"].float().cpu(), case["table"].cpu()
    q_all = case["q"].float().cpu()
    for row, length in enumerate(case["seq_lens"].tolist()):
        pages = table[row, : -(-length // page_size)].long()
        keys = k_all[pages].reshape(-1, Hkv, D)[:length]
        values = v_all[pages].reshape(-1, Hkv, D)[:length]
        q = q_all[row, : Hq * D].view(Hq, D)
        for head in range(Hq):
            scores = keys[:, head // group] @ q[head] / math.sqrt(D)
            out[row, head * D : (head + 1) * D] = torch.softmax(scores, dim=0) @ values[:, head // group]
    return out


def _static_entry():
    from kairyu_b200.kernels.build import load_library

    library = load_library("attention_decode_static")
    function = library.kb_attention_decode_mma_static
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    function.argtypes = [p, i, p, i, p, p, p, p, i, p, p, i, i, i, i, i, i, f, i, i, p]
    function.restype = i
    return library, function


def _call_static(function, case, out):
    return function(
        case["q"].data_ptr(), case["q"].stride(0), out.data_ptr(), out.stride(0), case["k"].data_ptr(), case["v"].data_ptr(),
        case["seq_lens"].data_ptr(), case["table"].data_ptr(), case["table"].shape[1], case["rows"].data_ptr(),
        case["tokens"].data_ptr(), case["count"], case["Hq"], case["Hkv"], case["D"], case["page_size"], case["num_pages"],
        1.0 / math.sqrt(case["D"]), 0, case["max_seq_len"], torch.cuda.current_stream().cuda_stream,
    )


def _call_ordinary(case, out):
    import kairyu_b200.kernels as kernels
    from kairyu_b200.engine.workspace import Workspace

    kernels.attention_decode_mma(
        case["q"], out, case["k"], case["v"], seq_lens=case["seq_lens"], block_table=case["table"], decode_rows=case["rows"],
        decode_tokens=case["tokens"], num_rows=case["count"], max_seq_len=case["max_seq_len"], num_q_heads=case["Hq"],
        scale=1.0 / math.sqrt(case["D"]), window=0, workspace=Workspace("cuda"),
    )


def test_static_entry_matches_the_ordinary_one_twice_in_a_row():
    library, function = _static_entry()
    assert library.kb_attention_decode_static_capacity() == 4 * 1024 * 1024
    # two calls in a row with different shapes: the second finds the first one's partials in the shared scratch
    cases = [_case([700, 1, 255, 257, 300], 8, 2, 64, 16, seed=1), _case([90, 513, 40], 6, 3, 32, 8, seed=2)]
    for case in cases:
        width = case["Hq"] * case["D"]
        expected = torch.zeros(case["count"], width, dtype=torch.bfloat16, device="cuda")
        _call_ordinary(case, expected)
        out = torch.zeros_like(expected)
        before = torch.cuda.memory_allocated()
        code = _call_static(function, case, out)
        assert code == 0
        assert torch.cuda.memory_allocated() == before  # nothing was taken from torch's allocator either
        torch.cuda.synchronize()
        assert float((out.float() - expected.float()).abs().max()) <= BF16_TOLERANCE
        assert float((out.float().cpu() - _plain_attention(case)).abs().max()) <= BF16_TOLERANCE
        assert float(out.float().abs().max()) > 0


def test_static_entry_refuses_what_its_scratch_cannot_hold():
    _, function = _static_entry()
    case = _case([64] * 4, 8, 2, 64, 16, seed=3)
    out = torch.zeros(case["count"], case["Hq"] * case["D"], dtype=torch.bfloat16, device="cuda")
    case["max_seq_len"] = 4_000_000  # 4 rows * 8 heads * 31,250 splits * 66 floats: far beyond 4 Mi floats
    assert _call_static(function, case, out) in (ERR_SCRATCH_TOO_SMALL, -1)
    case["max_seq_len"] = 300_000  # 2,344 splits: a valid grid, but 4.9 Mi floats
    assert _call_static(function, case, out) == ERR_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0  # nothing ran


def test_static_entry_refuses_bad_arguments_on_the_host():
    """A C caller gets an error code, not a fault on the device: a pointer off its 16-byte
    boundary, a page size of zero, an output narrower than its heads.  Nothing is launched."""
    _, function = _static_entry()
    case = _case([64] * 2, 4, 2, 32, 16, seed=4)
    out = torch.zeros(case["count"], case["Hq"] * case["D"], dtype=torch.bfloat16, device="cuda")
    good_q = case["q"]
    padded = torch.zeros(good_q.numel() + 8, dtype=torch.bfloat16, device="cuda")
    case["q"] = padded[1:][: good_q.numel()].view(good_q.shape)  # two bytes past a 16-byte boundary
    assert case["q"].data_ptr() % 16 == 2
    assert _call_static(function, case, out) == ERR_BAD_ARG
    case["q"] = good_q
    for key, value in (("page_size", 0), ("num_pages", 0)):
        broken = dict(case, **{key: value})
        assert _call_static(function, broken, out) == ERR_BAD_ARG
    narrow = torch.zeros(case["count"], case["Hq"] * case["D"] - 8, dtype=torch.bfloat16, device="cuda")
    assert _call_static(function, case, narrow) == ERR_BAD_ARG
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0
    assert _call_static(function, case, out) == 0  # and the same arguments put right are accepted
    torch.cuda.synchronize()
    assert float((out.float().cpu() - _plain_attention(case)).abs().max()) <= BF16_TOLERANCE
