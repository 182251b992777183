"""Each CUDA kernel alone against its plain torch statement (tests/torch_kernels.py),
at sizes other than the engine's: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd head groups, several page sizes.  Where
random data would hide a fault the inputs are built so that it shows (one key
among hundreds carries the whole softmax; keys at page, tile and split edges)."""

import math
from ctypes import c_int

import pytest
import torch

import torch_kernels as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def kernels():
    import kairyu_b200.kernels as k

    return k


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(a, b, atol, rtol=0.0):
    a = a.float().cpu()
    b = b.float().cpu()
    diff = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((diff <= bound).all()), f"max abs diff {diff.max().item():.3e} (atol {atol}, rtol {rtol})"


# ------------------------------------------------------------------ elementwise


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,T", [(331, 120, 17), (1000, 4096, 3)])
def test_embedding(dtype, V, H, T):
    table = rand(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32)
    out = torch.empty(T, H, dtype=torch.float32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().embedding(table.to(DEV), ids.to(DEV), out, flag)
    assert torch.equal(out.cpu(), table[ids.long()].float())
    assert int(flag.item()) == 0


def test_embedding_flags_a_bad_token():
    table = rand(50, 24).to(DEV)
    ids = torch.tensor([3, 50, -1], dtype=torch.int32, device=DEV)
    out = torch.full((3, 24), 7.0, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().embedding(table, ids, out, flag)
    assert int(flag.item()) == kernels().FLAG_BAD_TOKEN
    assert torch.equal(out[1:].cpu(), torch.zeros(2, 24))


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,T,eps", [(120, 9, 3e-6), (4096, 5, 1e-5), (96, 33, 1e-6)])
def test_rmsnorm_with_residual_sum(act, wdtype, H, T, eps):
    x = rand(T, H, seed=1)
    delta = rand(T, H, dtype=act, seed=2)
    w = (1 + 0.1 * rand(H, seed=3)).to(wdtype)
    # reference on the CPU
    x_ref = x.clone()
    out_ref = torch.empty(T, H, dtype=act)
    ref.rmsnorm(x_ref, w, eps, out_ref, delta=delta)
    x_dev = x.to(DEV)
    out = torch.empty(T, H, dtype=act, device=DEV)
    kernels().rmsnorm(x_dev, w.to(DEV), eps, out, delta=delta.to(DEV))
    close(x_dev, x_ref, 1e-6)  # the fp32 residual sum
    close(out, out_ref, 2e-6 if act == torch.float32 else 0.0, rtol=0.0 if act == torch.float32 else 1e-2)
    # without delta
    out2 = torch.empty(T, H, dtype=act, device=DEV)
    kernels().rmsnorm(x_dev, w.to(DEV), eps, out2)
    ref.rmsnorm(x_ref, w, eps, out_ref)
    close(out2, out_ref, 2e-6 if act == torch.float32 else 0.0, rtol=0.0 if act == torch.float32 else 1e-2)


@pytest.mark.parametrize("H", [96, 4096, 5120, 8192, 16384])
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_rmsnorm_rows_do_not_depend_on_how_many_there_are(H, act):
    """A few rows take larger blocks than many rows do; the sum of a row's squares is added in one order
    either way, so a row normed among 300 has the bits it has among 5."""
    x = rand(300, H, seed=8, scale=3.0)
    delta = rand(300, H, dtype=act, seed=9)
    w = (1 + 0.1 * rand(H, seed=10)).to(DEV)
    many_x, few_x = x.to(DEV), x[:5].to(DEV)
    many = torch.empty(300, H, dtype=act, device=DEV)
    few = torch.empty(5, H, dtype=act, device=DEV)
    kernels().rmsnorm(many_x, w, 1e-5, many, delta=delta.to(DEV))
    kernels().rmsnorm(few_x, w, 1e-5, few, delta=delta[:5].to(DEV))
    assert torch.equal(many[:5], few) and torch.equal(many_x[:5], few_x)


def test_rmsnorm_rows_leave_the_residual_alone():
    T, H = 12, 200
    x = rand(T, H, seed=4)
    delta = rand(T, H, seed=5)
    w = 1 + 0.1 * rand(H, seed=6)
    rows = torch.tensor([11, 0, 5], dtype=torch.int32)
    out_ref = torch.empty(3, H)
    ref.rmsnorm(x.clone(), w, 1e-5, out_ref, delta=delta, rows=rows)
    x_dev = x.to(DEV)
    out = torch.empty(3, H, device=DEV)
    kernels().rmsnorm(x_dev, w.to(DEV), 1e-5, out, delta=delta.to(DEV), rows=rows.to(DEV))
    assert torch.equal(x_dev.cpu(), x)
    close(out, out_ref, 2e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,I", [(7, 200), (3, 14336), (70, 160)])
def test_swiglu(dtype, T, I):
    gate_up = rand(T, 2 * I, dtype=dtype, seed=7, scale=2.0)
    out_ref = torch.empty(T, I, dtype=dtype)
    ref.swiglu(gate_up, out_ref)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    kernels().swiglu(gate_up.to(DEV), out)
    close(out, out_ref, 1e-6 if dtype == torch.float32 else 0.0, rtol=1e-6 if dtype == torch.float32 else 1e-2)


# ------------------------------------------------------------------ fp32 matrix product


@pytest.mark.parametrize("M,N,K", [(1, 331, 120), (65, 129, 17), (8, 4096, 4096), (130, 64, 200)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32_is_true_fp32(M, N, K, bias):
    x = rand(M, K, seed=8)
    w = rand(N, K, seed=9, scale=0.05)
    b = rand(N, seed=10) if bias else None
    expected = (x.double() @ w.double().t() + (b.double() if bias else 0)).float()
    out = torch.empty(M, N, device=DEV)
    kernels().linear(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, out)
    # fp32 accumulation error for K terms of magnitude ~0.05: far below TF32's 1e-3
    close(out, expected, 2e-6 * math.sqrt(K), rtol=1e-6)


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    x = rand(70, 200, seed=11)
    w = rand(300, 200, seed=12, scale=0.05)
    full = torch.empty(70, 300, device=DEV)
    kernels().linear(x.to(DEV), w.to(DEV), None, full)
    for start, stop in ((0, 1), (5, 6), (64, 70), (3, 68)):
        part = torch.empty(stop - start, 300, device=DEV)
        kernels().linear(x[start:stop].contiguous().to(DEV), w.to(DEV), None, part)
        assert torch.equal(part, full[start:stop])


@pytest.mark.parametrize("M,N,K", [(5, 96, 64), (64, 28672, 4096), (2048, 6144, 4096)])
def test_linear_bf16(M, N, K):
    x = rand(M, K, dtype=torch.bfloat16, seed=13)
    w = rand(N, K, dtype=torch.bfloat16, seed=14, scale=0.02)
    expected = x.float().to(DEV) @ w.float().to(DEV).t()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels().linear(x.to(DEV), w.to(DEV), None, out)
    close(out, expected, 2e-3 * math.sqrt(K / 64), rtol=1e-2)
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    kernels().linear(x.to(DEV), w.to(DEV), None, out32)
    close(out32, expected, 1e-4 * math.sqrt(K / 64), rtol=1e-4)


def test_products_stay_right_while_the_descriptor_table_turns_over(monkeypatch):
    """The tcgen05 product takes two encoded TMA descriptors per call from a bounded table.  With the
    table's limit at 4 every few calls turn it over; the descriptors of a call in progress must
    stay alive through that (they were once freed by a clear between the two look-ups)."""
    import kairyu_b200.kernels as module

    monkeypatch.setattr(module, "_TENSOR_MAP_LIMIT", 4)
    monkeypatch.setattr(module, "_tensor_maps", {})
    monkeypatch.setattr(module, "_tensor_maps_before", {})
    weights = [rand(N, K, dtype=torch.bfloat16, seed=60 + i, scale=0.05).to(DEV) for i, (N, K) in enumerate([(96, 64), (384, 96), (200, 160)])]
    for round_ in range(6):
        for w in weights:
            for M in (17, 33, 64, 40):
                x = rand(M, w.shape[1], dtype=torch.bfloat16, seed=70 + M + round_).to(DEV)
                out = torch.empty(M, w.shape[0], dtype=torch.float32, device=DEV)
                kernels().linear(x, w, None, out)
                close(out, x.float() @ w.float().t(), 1e-4 * math.sqrt(w.shape[1] / 64), rtol=1e-4)
    assert len(module._tensor_maps) <= 4


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(331, 144), (96, 64), (6144, 4096), (40, 16), (4096, 14336), (331, 120)])
@pytest.mark.parametrize("bias", [False, True])
def test_weight_streaming_product_for_few_rows(M, N, K, bias):
    """csrc/gemm_skinny.cu through ``linear`` (M <= 16): rows beyond M, weight rows beyond N and
    k beyond K (K not a multiple of 32) must not leak in."""
    x = rand(M, K, dtype=torch.bfloat16, seed=50)
    w = rand(N, K, dtype=torch.bfloat16, seed=51, scale=0.05)
    b = rand(N, dtype=torch.bfloat16, seed=52) if bias else None
    expected = x.float() @ w.float().t() + (b.float() if bias else 0)
    launches = kernels().launch_count
    for dtype, atol, rtol in ((torch.float32, 2e-4 * math.sqrt(K / 64), 1e-4), (torch.bfloat16, 4e-3 * math.sqrt(K / 64), 1e-2)):
        out = torch.full((M, N), 7.0, dtype=dtype, device=DEV)
        if K % 16 == 0:  # the kernel itself (``linear`` chooses it up to 8 rows)
            kernels().linear_weight_streaming(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, out)
        else:
            kernels().linear(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, out)
        close(out, expected, atol, rtol)
        if M <= 8:
            again = torch.full((M, N), 7.0, dtype=dtype, device=DEV)
            kernels().linear(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, again)
            if K % 16 == 0:
                assert torch.equal(again, out)  # ``linear`` ran the same kernel
    if K % 16 == 0:  # this package's kernel ran, not the library product (which takes the other sizes)
        assert kernels().launch_count == launches + (4 if M <= 8 else 2)


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(200, 144), (14336, 4096), (24, 64), (200, 120)])
def test_weight_streaming_product_with_the_gate_fused(M, I, K):
    x = rand(M, K, dtype=torch.bfloat16, seed=53)
    w = rand(2 * I, K, dtype=torch.bfloat16, seed=54, scale=0.05)
    y = x.float() @ w.float().t()
    g, u = y[:, :I], y[:, I:]
    expected = g / (1 + torch.exp(-g)) * u
    out = torch.full((M, I), 7.0, dtype=torch.bfloat16, device=DEV)
    from kairyu_b200.engine.workspace import Workspace

    kernels().linear_swiglu(x.to(DEV), w.to(DEV), out, Workspace(DEV))
    close(out, expected, 4e-3 * math.sqrt(K / 64), 1e-2)
    if K % 16 == 0:  # the weight-streaming kernel itself, which ``linear_swiglu`` chooses up to 8 rows
        direct = torch.full((M, I), 7.0, dtype=torch.bfloat16, device=DEV)
        kernels().linear_weight_streaming(x.to(DEV), w.to(DEV), None, direct, gated=True)
        close(direct, expected, 4e-3 * math.sqrt(K / 64), 1e-2)


def test_gated_product_for_many_rows_uses_the_two_kernel_path():
    from kairyu_b200.engine.workspace import Workspace

    M, I, K = 70, 160, 96
    x = rand(M, K, dtype=torch.bfloat16, seed=55)
    w = rand(2 * I, K, dtype=torch.bfloat16, seed=56, scale=0.05)
    expected = torch.empty(M, I, dtype=torch.bfloat16)
    ref.linear_swiglu(x, w, expected, None)
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    kernels().linear_swiglu(x.to(DEV), w.to(DEV), out, Workspace(DEV))
    close(out, expected, 2e-3, 1e-2)
    x32, w32 = x.float(), w.float()
    out32 = torch.empty(M, I, device=DEV)
    kernels().linear_swiglu(x32.to(DEV), w32.to(DEV), out32, Workspace(DEV))
    ref32 = torch.empty(M, I)
    ref.linear_swiglu(x32, w32, ref32, None)
    close(out32, ref32, 1e-5, 1e-5)


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K,gated", [(128, 64, False), (331, 144, False), (6144, 4096, False), (4096, 14336, False), (400, 200, True), (28672, 4096, True), (130, 72, True)])
@pytest.mark.parametrize("bias", [False, True])
def test_tcgen05_weight_streaming_product(M, N, K, gated, bias):
    """csrc/gemm_tc5.cu directly: TMA + tcgen05.mma with the accumulator in TMEM; weight rows beyond N,
    tokens beyond M and k beyond K come in as zeros; K split over blocks where N is small."""
    if gated and N == 28672 and bias:
        pytest.skip("one large gated case is enough")
    x = rand(M, K, dtype=torch.bfloat16, seed=60)
    w = rand(N, K, dtype=torch.bfloat16, seed=61, scale=0.05)
    b = rand(N, dtype=torch.bfloat16, seed=62) if bias else None
    y = x.float() @ w.float().t() + (b.float() if bias else 0)
    if gated:
        g, u = y[:, : N // 2], y[:, N // 2 :]
        y = g / (1 + torch.exp(-g)) * u
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dtype, atol, rtol in ((torch.float32, 3e-4 * math.sqrt(K / 64), 1e-4), (torch.bfloat16, 4e-3 * math.sqrt(K / 64), 1e-2)):
        out = torch.full(y.shape, 7.0, dtype=dtype, device=DEV)
        kernels()._gemm_tc5(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, out, gated=gated, flag=flag)
        close(out, y, atol, rtol)
    assert int(flag.item()) == 0


# ------------------------------------------------------------------ rope + cache write


def _rope_case(dtype, T, Hq, Hkv, D, page_size, qk_norm, rot_dim, seed):
    from kairyu_b200.parts.rope import rotary_tables

    g = torch.Generator().manual_seed(seed)
    max_pos = 300
    cos, sin = rotary_tables(rot_dim, 10000.0, None, max_pos)
    rows = 3
    row_ids = torch.sort(torch.randint(0, rows, (T,), generator=g)).values.to(torch.int32)
    positions = torch.randint(0, max_pos, (T,), generator=g).to(torch.int32)
    # distinct (row, position) pairs so that no two tokens write one slot
    seen = set()
    for t in range(T):
        while (int(row_ids[t]), int(positions[t])) in seen:
            positions[t] = (int(positions[t]) + 1) % max_pos
        seen.add((int(row_ids[t]), int(positions[t])))
    max_pages = -(-max_pos // page_size)
    num_pages = rows * max_pages + 1
    table = (torch.randperm(num_pages - 1, generator=g)[: rows * max_pages] + 1).view(rows, max_pages).to(torch.int32)
    write_from = torch.tensor([0, 40, 0], dtype=torch.int32)
    qkv = rand(T, (Hq + 2 * Hkv) * D, dtype=dtype, seed=seed + 1)
    qw = (1 + 0.1 * rand(D, seed=seed + 2)) if qk_norm else None
    kw = (1 + 0.1 * rand(D, seed=seed + 3)) if qk_norm else None
    return dict(cos=cos, sin=sin, row_ids=row_ids, positions=positions, table=table, write_from=write_from, qkv=qkv, qw=qw, kw=kw, num_pages=num_pages)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(
    "Hq,Hkv,D,page_size,qk_norm,rot_dim",
    [(4, 2, 16, 16, False, 16), (6, 3, 32, 8, True, 32), (5, 1, 48, 16, True, 48), (32, 8, 128, 16, False, 128), (3, 3, 80, 4, True, 32),
     # heads of 128 in bf16 with many tokens: the kernel that gives a token eight lanes of 16 bytes
     (32, 8, 128, 16, True, 128), (5, 1, 128, 8, True, 128), (9, 3, 128, 32, False, 128),
     # and heads of 64: four lanes a head, sixteen groups of them a token
     (32, 8, 64, 16, True, 64), (32, 8, 64, 16, False, 64), (7, 1, 64, 8, True, 64), (100, 14, 64, 32, False, 64)],
)
@pytest.mark.parametrize("T", [37, 301])  # 301: the many-token kernels (full rotation, heads up to 128), with a ragged end
def test_qk_norm_rope_kv_write(dtype, Hq, Hkv, D, page_size, qk_norm, rot_dim, T):
    case = _rope_case(dtype, T, Hq, Hkv, D, page_size, qk_norm, rot_dim, seed=20)
    kc_ref = torch.zeros(case["num_pages"], page_size, Hkv, D, dtype=dtype)
    vc_ref = torch.zeros_like(kc_ref)
    qkv_ref = case["qkv"].clone()
    common = dict(positions=case["positions"], row_ids=case["row_ids"], eps=1e-6)
    ref.qk_norm_rope_kv_write(
        qkv_ref, Hq, Hkv, D, q_norm_weight=case["qw"], k_norm_weight=case["kw"], cos=case["cos"], sin=case["sin"],
        block_table=case["table"], write_from=case["write_from"], k_cache=kc_ref, v_cache=vc_ref, **common,
    )
    to = lambda t: None if t is None else t.to(DEV)
    qkv = case["qkv"].to(DEV)
    kc = torch.zeros_like(kc_ref, device=DEV)
    vc = torch.zeros_like(kc_ref, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().qk_norm_rope_kv_write(
        qkv, Hq, Hkv, D, positions=to(case["positions"]), row_ids=to(case["row_ids"]), q_norm_weight=to(case["qw"]),
        k_norm_weight=to(case["kw"]), eps=1e-6, cos=to(case["cos"]), sin=to(case["sin"]), block_table=to(case["table"]),
        write_from=to(case["write_from"]), k_cache=kc, v_cache=vc, flag=flag,
    )
    assert int(flag.item()) == 0
    # bf16 results are compared to a hundredth of their size, plus the absolute term of the 32-bit branch: where
    # a * cos and b * sin cancel to the last bits (an output of 1.8e-7 from products of size 1 in the case of
    # 100 + 14 heads), a fused multiply-add and two rounded products differ by the rounding of one product,
    # which is more than a hundredth of such an output and far below anything the model can see
    atol, rtol = (3e-6, 1e-6) if dtype == torch.float32 else (3e-6, 1e-2)
    q_size, kv_size = Hq * D, Hkv * D
    close(qkv[:, : q_size + kv_size], qkv_ref[:, : q_size + kv_size], atol, rtol)
    assert torch.equal(qkv[:, q_size + kv_size :].cpu(), qkv_ref[:, q_size + kv_size :])  # v untouched
    close(kc, kc_ref, atol, rtol)
    assert torch.equal(vc.cpu(), vc_ref)
    # positions below write_from wrote nothing: the slots of row 1 below position 40 stay zero
    written = (kc_ref.abs().sum(dim=(2, 3)) > 0)
    assert torch.equal((kc.cpu().float().abs().sum(dim=(2, 3)) > 0), written)


@pytest.mark.parametrize("Hq,Hkv,D,page_size,K", [(4, 2, 16, 16, 64), (5, 1, 48, 16, 112), (32, 8, 128, 16, 4096), (3, 3, 80, 4, 96)])
@pytest.mark.parametrize("T", [1, 8, 13])
@pytest.mark.parametrize("bias", [False, True])
def test_product_with_rotation_and_cache_write_in_its_epilogue(Hq, Hkv, D, page_size, K, T, bias):
    """``linear_rope`` against the product in fp32, then the plain rotation and cache write: the q
    columns of the output, the key and value pages, nothing written below ``write_from``."""
    case = _rope_case(torch.bfloat16, T, Hq, Hkv, D, page_size, False, D, seed=30)
    N = (Hq + 2 * Hkv) * D
    x = rand(T, K, dtype=torch.bfloat16, seed=31)
    w = rand(N, K, dtype=torch.bfloat16, seed=32, scale=0.05)
    b = rand(N, dtype=torch.bfloat16, seed=33) if bias else None
    product = x.float() @ w.float().t() + (b.float() if bias else 0)
    kc_ref = torch.zeros(case["num_pages"], page_size, Hkv, D)
    vc_ref = torch.zeros_like(kc_ref)
    placement = dict(positions=case["positions"], row_ids=case["row_ids"], block_table=case["table"], write_from=case["write_from"])
    ref.qk_norm_rope_kv_write(product, Hq, Hkv, D, cos=case["cos"], sin=case["sin"], k_cache=kc_ref, v_cache=vc_ref, **placement)
    to = lambda t: None if t is None else t.to(DEV)
    out = torch.full((T, N), 7.0, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(kc_ref.shape, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    heads = dict(num_q_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    assert kernels().linear_rope_ok(to(x), to(w), to(b), out, cos=to(case["cos"]), k_cache=kc, **heads)
    kernels().linear_rope(
        to(x), to(w), to(b), out, cos=to(case["cos"]), sin=to(case["sin"]), k_cache=kc, v_cache=vc, flag=flag,
        **heads, **{name: to(t) for name, t in placement.items()},
    )
    assert int(flag.item()) == 0
    atol, rtol = 4e-3 * math.sqrt(K / 64) + 4e-3, 1e-2
    close(out[:, : Hq * D], product[:, : Hq * D], atol, rtol)
    assert bool((out[:, Hq * D :] == 7.0).all())  # k and v go to the cache only
    close(kc, kc_ref, atol, rtol)
    close(vc, vc_ref, atol, rtol)
    written = kc_ref.abs().sum(dim=(2, 3)) > 0
    assert torch.equal(kc.cpu().float().abs().sum(dim=(2, 3)) > 0, written)
    assert torch.equal(vc.cpu().float().abs().sum(dim=(2, 3)) > 0, vc_ref.abs().sum(dim=(2, 3)) > 0)


def test_rope_flags_a_position_outside_the_table():
    from kairyu_b200.parts.rope import rotary_tables

    cos, sin = rotary_tables(16, 10000.0, None, 8)
    qkv = rand(2, 4 * 16).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().qk_norm_rope_kv_write(
        qkv, 2, 1, 16, positions=torch.tensor([3, 8], dtype=torch.int32, device=DEV),
        row_ids=torch.zeros(2, dtype=torch.int32, device=DEV), cos=cos.to(DEV), sin=sin.to(DEV), flag=flag,
    )
    assert int(flag.item()) == kernels().FLAG_BAD_POS


@pytest.mark.parametrize("M,H,N,bias", [(1, 64, 48, False), (8, 4096, 6144, False), (5, 160, 208, True), (16, 1024, 512, True), (9, 96, 4096, False)])
def test_rmsnorm_split_between_two_products(M, H, N, bias):
    """fold: a product adds its result to the residual and leaves weighted rows and sums of squares;
    scale: the next product finishes the norm in its epilogue (plain and gated).  Against the plain statement."""
    k = kernels()
    K0 = 320  # inner size of the folding product
    g = torch.Generator().manual_seed(50 + M)
    x0 = (torch.randn(M, K0, generator=g) * 0.5).bfloat16()
    w0 = (torch.randn(H, K0, generator=g) * 0.05).bfloat16()
    b0 = (torch.randn(H, generator=g) * 0.1).bfloat16() if bias else None
    residual = torch.randn(M, H, generator=g) * 2.0
    residual[0, 3] = 40.0  # an outlier channel, as residual streams have
    norm_w = 1.0 + 0.1 * torch.randn(H, generator=g)
    w1 = (torch.randn(N, H, generator=g) * 0.05).bfloat16()
    b1 = (torch.randn(N, generator=g) * 0.1).bfloat16() if bias else None
    eps = 1e-5
    # plain: r' = r + x0 W0^T (+b0); y = rmsnorm(r') * g; out = y W1^T (+ b1)
    r_new = residual + x0.float() @ w0.float().t() + (b0.float() if bias else 0.0)
    y = r_new * torch.rsqrt(r_new.pow(2).mean(-1, keepdim=True) + eps) * norm_w
    expected = y @ w1.float().t() + (b1.float() if bias else 0.0)
    half = N // 2
    expected_gated = torch.nn.functional.silu(expected[:, :half] - (b1.float()[:half] if bias else 0.0)) * (expected[:, half:] - (b1.float()[half:] if bias else 0.0))

    dev_res = residual.to(DEV)
    blocks = k.skinny_blocks(M, H)
    fold = k.ResidualNorm(
        dev_res, norm_w.to(DEV), eps, torch.empty(M, H, dtype=torch.bfloat16, device=DEV),
        torch.full((blocks, 16), float("nan"), device=DEV),
    )
    k.linear(x0.to(DEV), w0.to(DEV), b0.to(DEV) if bias else None, None, fold=fold)
    close(dev_res, r_new, 2e-3)
    pre = fold.result()
    sums = pre.sumsq[:, :M].sum(0).cpu()
    close(sums, r_new.pow(2).sum(-1), 1e-2, rtol=1e-4)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    k.linear(pre, w1.to(DEV), b1.to(DEV) if bias else None, out)
    close(out, expected, 3e-2, rtol=2e-2)
    if N % 2 == 0:
        gated = torch.empty(M, half, dtype=torch.bfloat16, device=DEV)
        k.linear_swiglu(pre, w1.to(DEV), gated, None)
        # an error e in gate or up shows as about e * |the other factor| in the product
        gate, up = expected[:, :half] - (b1.float()[:half] if bias else 0.0), expected[:, half:] - (b1.float()[half:] if bias else 0.0)
        bound = (3e-2 + 2e-2 * gate.abs()) * (1.0 + up.abs()) + (3e-2 + 2e-2 * up.abs()) * (1.0 + gate.abs())
        assert bool(((gated.float().cpu() - expected_gated).abs() <= bound).all())


def test_patch_tokens_takes_ids_from_the_device_and_flags_a_bad_source():
    ids = torch.tensor([5, 0, 7, 0, 9], dtype=torch.int32, device=DEV)
    source = torch.tensor([-1, 2, -1, 0, -1], dtype=torch.int32, device=DEV)
    sampled = torch.tensor([41, 42, 43], dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().patch_tokens(ids, source, sampled, flag)
    assert ids.cpu().tolist() == [5, 43, 7, 41, 9] and int(flag.item()) == 0
    expected = torch.tensor([5, 0, 7, 0, 9], dtype=torch.int32)
    ref.patch_tokens(expected, source.cpu(), sampled.cpu())
    assert expected.tolist() == ids.cpu().tolist()
    source[1] = 3  # outside the sampled tensor: flagged, the id stays
    kernels().patch_tokens(ids, source, sampled, flag)
    assert int(flag.item()) == kernels().FLAG_BAD_ROW and ids.cpu().tolist() == [5, 43, 7, 41, 9]


# ------------------------------------------------------------------ attention


def _attention_case(dtype, Hq, Hkv, D, page_size, seq_lens, chunk_lens, seed, hot=None):
    """A cache filled with random keys and values for `len(seq_lens)` requests and
    the queries of their last `chunk_lens[i]` positions.  ``hot`` = (row, key
    position): that key is made to dominate the softmax of every later query of
    the row, and its value is set apart, so a kernel that skips or misplaces it
    returns something visibly different."""
    g = torch.Generator().manual_seed(seed)
    rows = len(seq_lens)
    max_pages = max(-(-s // page_size) for s in seq_lens) + 1
    num_pages = rows * max_pages + 3
    perm = torch.randperm(num_pages - 1, generator=g) + 1
    table = torch.full((rows, max_pages), -1, dtype=torch.int32)
    # Everything no request holds is NaN, but for page 0, which the cache manager keeps
    # aside (and finite) for rows that stand in for absent ones: a kernel that lets a
    # stale row into its sums shows it.
    kc = torch.full((num_pages, page_size, Hkv, D), float("nan"))
    kc[0] = 0.0
    vc = kc.clone()
    used = 0
    for r, s in enumerate(seq_lens):
        n = -(-s // page_size)
        table[r, :n] = perm[used : used + n].to(torch.int32)
        used += n
        for j in range(s):
            page = int(table[r, j // page_size])
            kc[page, j % page_size] = torch.randn(Hkv, D, generator=g) * 0.5
            vc[page, j % page_size] = torch.randn(Hkv, D, generator=g)
    tokens = sum(chunk_lens)
    q = torch.randn(tokens, Hq * D, generator=g) * 0.5
    positions, row_ids, qo = [], [], [0]
    for r, (s, c) in enumerate(zip(seq_lens, chunk_lens)):
        positions += list(range(s - c, s))
        row_ids += [r] * c
        qo.append(qo[-1] + c)
    if hot is not None:
        r, key = hot
        page = int(table[r, key // page_size])
        direction = torch.randn(D, generator=g)
        direction = direction / direction.norm()
        kc[page, key % page_size] = direction * 16.0
        vc[page, key % page_size] = 25.0
        for t in range(qo[r], qo[r + 1]):
            q[t] = (direction * 16.0).repeat(Hq)
    return dict(
        q=q.to(dtype), kc=kc.to(dtype), vc=vc.to(dtype), table=table,
        positions=torch.tensor(positions, dtype=torch.int32), row_ids=torch.tensor(row_ids, dtype=torch.int32),
        qo=torch.tensor(qo, dtype=torch.int32), seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
    )


def _reference_attention(case, Hq, scale, window):
    out = torch.empty(case["q"].shape[0], case["q"].shape[1])
    ref.paged_attention_generic(
        case["q"].float(), out, case["kc"].float(), case["vc"].float(), positions=case["positions"],
        row_ids=case["row_ids"], block_table=case["table"], num_q_heads=Hq, scale=scale, window=window,
    )
    return out


GEOMETRIES = [
    (4, 2, 16, 16), (6, 3, 32, 8), (5, 1, 48, 16), (32, 8, 128, 16), (8, 2, 80, 32), (2, 2, 256, 16), (6, 1, 64, 4),
    (6, 2, 192, 8), (4, 1, 64, 64), (4, 2, 128, 128), (3, 3, 64, 32),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,page_size", GEOMETRIES)
@pytest.mark.parametrize("window", [0, 37])
def test_generic_attention(dtype, Hq, Hkv, D, page_size, window):
    case = _attention_case(dtype, Hq, Hkv, D, page_size, [70, 1, 130], [70, 1, 9], seed=30)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    out = torch.empty(case["q"].shape, dtype=dtype, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().paged_attention_generic(
        case["q"].to(DEV), out, case["kc"].to(DEV), case["vc"].to(DEV), positions=case["positions"].to(DEV),
        row_ids=case["row_ids"].to(DEV), block_table=case["table"].to(DEV), num_q_heads=Hq, scale=scale, window=window, flag=flag,
    )
    assert int(flag.item()) == 0
    close(out, expected, 2e-5 if dtype == torch.float32 else 2e-2)


def _run_mma(case, Hq, scale, window, workspace):
    """Both tensor-core kernels over a case: tiles for rows with several tokens, split-KV for single-token rows."""
    k = kernels()
    qo = case["qo"].tolist()
    tile_rows, tile_starts, decode_rows, decode_tokens = [], [], [], []
    for r in range(len(qo) - 1):
        count = qo[r + 1] - qo[r]
        if count == 1:
            decode_rows.append(r)
            decode_tokens.append(qo[r])
        else:
            for start in range(0, count, k.attention_prefill_tile_rows(case["kc"].shape[-1])):
                tile_rows.append(r)
                tile_starts.append(start)
    dev = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    q = case["q"].to(DEV)
    out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
    kc, vc = case["kc"].to(DEV), case["vc"].to(DEV)
    if tile_rows:
        k.attention_prefill_mma(
            q, out, kc, vc, qo_indptr=case["qo"].to(DEV), seq_lens=case["seq_lens"].to(DEV), block_table=case["table"].to(DEV),
            tile_rows=dev(tile_rows), tile_starts=dev(tile_starts), num_tiles=len(tile_rows), num_q_heads=Hq, scale=scale, window=window,
        )
    if decode_rows:
        k.attention_decode_mma(
            q, out, kc, vc, seq_lens=case["seq_lens"].to(DEV), block_table=case["table"].to(DEV), decode_rows=dev(decode_rows),
            decode_tokens=dev(decode_tokens), num_rows=len(decode_rows), max_seq_len=int(case["seq_lens"].max()),
            num_q_heads=Hq, scale=scale, window=window, workspace=workspace,
        )
    return out


@pytest.fixture
def workspace():
    from kairyu_b200.engine.workspace import Workspace

    return Workspace(DEV)


@pytest.mark.parametrize("Hq,Hkv,D,page_size", GEOMETRIES)
@pytest.mark.parametrize("window", [0, 37, 300])
def test_mma_attention_random(Hq, Hkv, D, page_size, window, workspace):
    # rows: a whole prompt of several tiles, a portion in the middle of a long request,
    # decode rows at 1, just under/over a split (256) and further, a 2-token portion
    seq_lens = [150, 400, 1, 255, 257, 700, 66]
    chunk_lens = [150, 70, 1, 1, 1, 1, 2]
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, chunk_lens, seed=31)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    out = _run_mma(case, Hq, scale, window, workspace)
    close(out, expected, 2e-2)


@pytest.mark.parametrize("Hq,Hkv,D,page_size", [(8, 2, 64, 16), (32, 8, 128, 16), (6, 2, 192, 8), (2, 1, 256, 64)])
@pytest.mark.parametrize("num_splits", [1, 2, 3, 7, 8, 9, 16])
@pytest.mark.parametrize("window", [0, 333])
def test_decode_attention_streams_many_tiles_through_its_ring(Hq, Hkv, D, page_size, num_splits, window, workspace):
    """Few splits and long rows: every block of the TMA-fed kernel refills its stages several times."""
    seq_lens = [1000, 700, 257, 64, 1]
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, [1] * len(seq_lens), seed=35)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
    rows = torch.arange(len(seq_lens), dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels().attention_decode_mma(
        case["q"].to(DEV), out, case["kc"].to(DEV), case["vc"].to(DEV), seq_lens=case["seq_lens"].to(DEV),
        block_table=case["table"].to(DEV), decode_rows=rows, decode_tokens=rows, num_rows=len(seq_lens), max_seq_len=max(seq_lens),
        num_q_heads=Hq, scale=scale, window=window, workspace=workspace, flag=flag, num_splits=num_splits,
    )
    assert int(flag.item()) == 0
    close(out, expected, 2e-2)


@pytest.mark.parametrize("Hq,Hkv,page_size", [(8, 2, 16), (32, 8, 16), (6, 3, 8), (4, 1, 64), (2, 2, 128)])
@pytest.mark.parametrize("num_splits", [1, 3, 8])
@pytest.mark.parametrize("window", [0, 333])
def test_decode_attention_fetches_keys_and_values_in_one_copy(Hq, Hkv, page_size, num_splits, window, workspace):
    """Head size 64 with the values a fixed distance behind the keys in one allocation (as the cache storage
    lays them out): one strided copy brings both.  Values that differ from the keys in every element, so
    that a mix-up of the two halves of a stage shows; the same bits as with two allocations."""
    D = 64
    seq_lens = [1000, 700, 257, 64, 1]
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, [1] * len(seq_lens), seed=41)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    both = torch.stack([case["kc"], case["vc"]]).to(DEV)
    rows = torch.arange(len(seq_lens), dtype=torch.int32, device=DEV)
    k = kernels()
    assert k._joined_cache_map(both[0], both[1]) != 0
    swapped = torch.stack([case["vc"], case["kc"]]).to(DEV)  # the values BEFORE the keys: no such copy, two maps
    assert k._joined_cache_map(swapped[1], swapped[0]) == 0
    outs = []
    for kc, vc in ((both[0], both[1]), (swapped[1], swapped[0])):
        out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        k.attention_decode_mma(
            case["q"].to(DEV), out, kc, vc, seq_lens=case["seq_lens"].to(DEV), block_table=case["table"].to(DEV),
            decode_rows=rows, decode_tokens=rows, num_rows=len(seq_lens), max_seq_len=max(seq_lens), num_q_heads=Hq,
            scale=scale, window=window, workspace=workspace, flag=flag, num_splits=num_splits,
        )
        assert int(flag.item()) == 0
        close(out, expected, 2e-2)
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("joined", [True, False])
@pytest.mark.parametrize("window", [0, 333])
@pytest.mark.parametrize("D,count", [(64, 60), (128, 40)])
def test_decode_attention_of_a_grid_too_large_for_one_wave(joined, window, D, count, workspace):
    """60 rows x 8 KV heads at head size 64, 40 at 128: more blocks than fit the SMs at once with the
    usual ring, so the launcher takes the one with a stage less and a block more an SM; rows of 1 to 900
    keys, so that the ring wraps several times in the long ones."""
    Hq, Hkv, page_size = 16, 8, 16
    if D != 64 and joined:
        pytest.skip("keys and values share a copy at head size 64 only")
    seq_lens = [1 + (37 * r) % 900 for r in range(count)]
    seq_lens[7], seq_lens[8] = 900, 64
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, [1] * len(seq_lens), seed=43)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    both = torch.stack([case["kc"], case["vc"]] if joined else [case["vc"], case["kc"]]).to(DEV)
    kc, vc = (both[0], both[1]) if joined else (both[1], both[0])
    k = kernels()
    assert (k._joined_cache_map(kc, vc) != 0) == joined
    resident = k._fn("attention_decode_tma", "kb_attention_decode_tma_splits", [c_int] * 4)
    assert resident(len(seq_lens), Hkv, D, max(seq_lens)) == 1  # no room for a second split: the grid is crowded
    rows = torch.arange(len(seq_lens), dtype=torch.int32, device=DEV)
    out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.attention_decode_mma(
        case["q"].to(DEV), out, kc, vc, seq_lens=case["seq_lens"].to(DEV), block_table=case["table"].to(DEV),
        decode_rows=rows, decode_tokens=rows, num_rows=len(seq_lens), max_seq_len=max(seq_lens), num_q_heads=Hq,
        scale=scale, window=window, workspace=workspace, flag=flag,
    )
    assert int(flag.item()) == 0
    close(out, expected, 2e-2)


def _run_prefill(case, Hq, scale, window, workspace, num_splits, max_seq_len=0, two_tiles=None):
    k = kernels()
    qo = case["qo"].tolist()
    tile_rows, tile_starts, wide_rows, wide_starts = [], [], [], []
    for r in range(len(qo) - 1):
        for start in range(0, qo[r + 1] - qo[r], k.attention_prefill_tile_rows(case["kc"].shape[-1])):
            tile_rows.append(r)
            tile_starts.append(start)
        for start in range(0, qo[r + 1] - qo[r], 256):
            wide_rows.append(r)
            wide_starts.append(start)
    dev = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    wide = (len(wide_rows), dev(wide_rows), dev(wide_starts)) if two_tiles is not None else None
    out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    k.attention_prefill_mma(
        case["q"].to(DEV), out, case["kc"].to(DEV), case["vc"].to(DEV), qo_indptr=case["qo"].to(DEV), seq_lens=case["seq_lens"].to(DEV),
        block_table=case["table"].to(DEV), tile_rows=dev(tile_rows), tile_starts=dev(tile_starts), num_tiles=len(tile_rows),
        num_q_heads=Hq, scale=scale, window=window, flag=flag, workspace=workspace, num_splits=num_splits, max_seq_len=max_seq_len,
        wide_tiles=wide, two_tiles=two_tiles,
    )
    assert int(flag.item()) == 0
    return out


@pytest.mark.parametrize("Hq,Hkv,page_size", [(8, 2, 16), (32, 8, 16), (4, 4, 8), (6, 1, 32), (4, 2, 128)])
@pytest.mark.parametrize("window", [0, 37, 333])
def test_prefill_attention_two_query_tiles_a_block(Hq, Hkv, page_size, window, workspace):
    """The kernel that walks two 128-query tiles over 128-key tiles: a whole prompt of five tiles (the
    last block has one tile, and that ragged), a portion that starts at an odd position deep in a
    request, a portion of exactly 256, a short one and a 2-token one; with windows shorter and longer
    than a key tile (tile B starts later than tile A, whole key tiles lie before the window)."""
    D = 128
    seq_lens = [600, 1301, 256, 777, 300]
    chunk_lens = [600, 391, 256, 100, 2]
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, chunk_lens, seed=39)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    out = _run_prefill(case, Hq, scale, window, workspace, 1, two_tiles=True)
    close(out, expected, 2e-2)
    assert torch.equal(out, _run_prefill(case, Hq, scale, window, workspace, 1, two_tiles=True))


@pytest.mark.parametrize("hot_key", [0, 127, 128, 129, 700, 1023, 1024, 1150, 1279])
def test_prefill_attention_two_tiles_finds_one_far_key(hot_key, workspace):
    """One key among 1,280 carries the softmax of the last 300 queries, wherever it lies in a key tile."""
    Hq, Hkv, D, page_size = 8, 2, 128, 16
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, [1280], [300], seed=40, hot=(0, hot_key))
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, 0)
    visible = [t for t in range(300) if 1280 - 300 + t >= hot_key]
    assert float(expected[visible].min()) > 24.0
    out = _run_prefill(case, Hq, scale, 0, workspace, 1, two_tiles=True)
    close(out, expected, 2e-2, rtol=1e-2)


@pytest.mark.parametrize("Hq,Hkv,D,page_size", [(8, 2, 64, 16), (32, 8, 128, 16), (4, 1, 128, 64), (6, 3, 64, 8)])
@pytest.mark.parametrize("num_splits", [2, 3, 8])
@pytest.mark.parametrize("window", [0, 333])
def test_prefill_attention_with_the_keys_split_over_blocks(Hq, Hkv, D, page_size, num_splits, window, workspace):
    """Portions of long requests whose keys several blocks share: a portion deep in a request, one
    whose last tile is ragged, a fresh short prompt (fewer key tiles than splits: blocks without
    keys), a 2-token portion."""
    seq_lens = [900, 1300, 150, 700]
    chunk_lens = [200, 131, 150, 2]
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, chunk_lens, seed=37)
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    out = _run_prefill(case, Hq, scale, window, workspace, num_splits)
    close(out, expected, 2e-2)
    again = _run_prefill(case, Hq, scale, window, workspace, num_splits)
    assert torch.equal(out, again)  # the splits are combined in order, not as they arrive


@pytest.mark.parametrize("hot_key", [0, 63, 64, 500, 1023, 1024, 1900])
def test_prefill_attention_split_finds_one_far_key(hot_key, workspace):
    """One key among 2,000 carries the softmax of a 128-token portion, whichever block's share it lies in;
    the number of splits is the kernel's own choice (a lone tile of few heads: as many as it takes)."""
    Hq, Hkv, D, page_size = 8, 2, 128, 16
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, [2000], [128], seed=38, hot=(0, hot_key))
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, 0)
    visible = [t for t in range(128) if 2000 - 128 + t >= hot_key]
    assert float(expected[visible].min()) > 24.0  # the reference itself is dominated by that key
    assert kernels()._fn("attention_prefill_tc5", "kb_attention_prefill_tc5_splits", [c_int] * 4)(D, Hq, 1, 2000) > 1
    out = _run_prefill(case, Hq, scale, 0, workspace, None, max_seq_len=2000)
    close(out, expected, 2e-2, rtol=1e-2)


@pytest.mark.parametrize("num_splits", [None, 1, 5])
def test_decode_attention_long_context(num_splits, workspace):
    """Thousands of keys: tens of ring refills per block, a hot key far back, a window over most of it."""
    Hq, Hkv, D, page_size = 8, 2, 128, 16
    seq_lens = [5000, 4097, 3]
    for window, hot in ((0, (0, 77)), (4500, (1, 1000))):
        case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, seq_lens, [1] * 3, seed=36, hot=hot)
        scale = 1.0 / math.sqrt(D)
        expected = _reference_attention(case, Hq, scale, window)
        assert float(expected[hot[0]].min()) > 24.0
        out = torch.zeros(case["q"].shape, dtype=torch.bfloat16, device=DEV)
        rows = torch.arange(3, dtype=torch.int32, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        kernels().attention_decode_mma(
            case["q"].to(DEV), out, case["kc"].to(DEV), case["vc"].to(DEV), seq_lens=case["seq_lens"].to(DEV),
            block_table=case["table"].to(DEV), decode_rows=rows, decode_tokens=rows, num_rows=3, max_seq_len=max(seq_lens),
            num_q_heads=Hq, scale=scale, window=window, workspace=workspace, flag=flag, num_splits=num_splits,
        )
        assert int(flag.item()) == 0
        close(out, expected, 2e-2, rtol=1e-2)


@pytest.mark.parametrize("hot_key", [0, 15, 16, 17, 63, 64, 127, 128, 129, 255, 256, 257, 511, 512, 640, 699])
@pytest.mark.parametrize("chunk", [1, 2, 61])
def test_mma_attention_finds_one_far_key(hot_key, chunk, workspace):
    """One key among 700 carries the softmax; the output must be its value."""
    Hq, Hkv, D, page_size = 8, 2, 64, 16
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, [700, 300], [chunk, 1], seed=32, hot=(0, hot_key))
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, 0)
    visible = [t for t in range(chunk) if 700 - chunk + t >= hot_key]
    assert visible and float(expected[visible].min()) > 24.0  # the reference itself is dominated by that key
    out = _run_mma(case, Hq, scale, 0, workspace)
    close(out, expected, 2e-2, rtol=1e-2)


@pytest.mark.parametrize("window,hot_key,inside", [(64, 636, True), (64, 635, False), (300, 400, True), (300, 399, False)])
@pytest.mark.parametrize("Hq,Hkv,D,page_size", [(4, 4, 32, 8), (4, 2, 64, 16), (8, 1, 128, 64)])
def test_mma_attention_window_edge(window, hot_key, inside, Hq, Hkv, D, page_size, workspace):
    """The dominating key sits exactly on, or one before, the window's edge of the last query."""
    case = _attention_case(torch.bfloat16, Hq, Hkv, D, page_size, [700], [1], seed=33, hot=(0, hot_key))
    scale = 1.0 / math.sqrt(D)
    expected = _reference_attention(case, Hq, scale, window)
    assert (float(expected.min()) > 24.0) == inside
    out = _run_mma(case, Hq, scale, window, workspace)
    close(out, expected, 2e-2, rtol=1e-2)
    generic = torch.empty(case["q"].shape, dtype=torch.bfloat16, device=DEV)
    kernels().paged_attention_generic(
        case["q"].to(DEV), generic, case["kc"].to(DEV), case["vc"].to(DEV), positions=case["positions"].to(DEV),
        row_ids=case["row_ids"].to(DEV), block_table=case["table"].to(DEV), num_q_heads=Hq, scale=scale, window=window,
    )
    close(generic, expected, 2e-2, rtol=1e-2)


def test_attention_flags_a_page_outside_the_pool():
    case = _attention_case(torch.float32, 2, 1, 16, 16, [40], [1], seed=34)
    table = case["table"].clone()
    table[0, 1] = 10_000
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(case["q"].shape, device=DEV)
    kernels().paged_attention_generic(
        case["q"].to(DEV), out, case["kc"].to(DEV), case["vc"].to(DEV), positions=case["positions"].to(DEV),
        row_ids=case["row_ids"].to(DEV), block_table=table.to(DEV), num_q_heads=2, scale=0.25, flag=flag,
    )
    assert int(flag.item()) == kernels().FLAG_BAD_PAGE


# ------------------------------------------------------------------ sampling


@pytest.mark.parametrize("n,V", [(1, 331), (5, 128256), (64, 1000)])
def test_argmax(n, V):
    logits = rand(n, V, seed=40)
    logits[0, V - 1] = 50.0
    if n > 1:
        logits[1, 7] = logits[1, 300] = 60.0  # a tie: the first index wins
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    kernels().argmax(logits.to(DEV), out)
    assert out.cpu().tolist() == logits.argmax(dim=-1).tolist()
    if n > 1:
        assert int(out[1]) == 7


def test_edit_logits():
    logits = rand(3, 50, seed=41)
    rows = torch.tensor([0, 0, 2, 1], dtype=torch.int32)
    tokens = torch.tensor([4, 9, 4, 49], dtype=torch.int32)
    mul = torch.tensor([1.3, 1.0, 0.7, 1.0])
    sub = torch.tensor([0.0, 0.9, 0.2, 0.0])
    mask = torch.tensor([0, 0, 0, 1], dtype=torch.int32)
    expected = logits.clone()
    ref.edit_logits(expected, rows, tokens, mul, sub, mask)
    dev = logits.to(DEV)
    kernels().edit_logits(dev, rows.to(DEV), tokens.to(DEV), mul.to(DEV), sub.to(DEV), mask.to(DEV))
    assert math.isinf(float(dev[1, 49])) and float(dev[1, 49]) < 0
    dev[1, 49] = expected[1, 49] = 0.0
    close(dev, expected, 1e-6)


@pytest.mark.parametrize("n,V,k", [(3, 331, 5), (6, 128256, 20), (2, 1000, 0), (1, 7, 12), (2, 300000, 3)])
def test_logprob_report(n, V, k):
    """Log-softmax of the chosen token and the k largest, against torch.log_softmax / topk in fp32;
    ties go to the lower index; more asked for than the vocabulary holds marks the rest absent."""
    logits = rand(n, V, seed=44) * 4.0
    if V > 300:
        logits[0, 7] = logits[0, 300] = 30.0  # a tie at the top
        logits[n - 1, V - 1] = 25.0
    rows = list(range(n - 1, -1, -1))[: max(1, n - 1)]  # another order than the rows', and not all of them
    tokens = torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(45), dtype=torch.int32)
    values = torch.full((len(rows), k + 1), float("nan"), device=DEV)
    indices = torch.full((len(rows), k), -7, dtype=torch.int32, device=DEV)
    kernels().logprob_report(
        logits.to(DEV), torch.tensor(rows, dtype=torch.int32, device=DEV), tokens.to(DEV), k, values, indices, tokens_by_row=True
    )
    values, indices = values.cpu(), indices.cpu()
    logp = torch.log_softmax(logits.double(), dim=-1)
    have = min(k, V)
    for place, row in enumerate(rows):
        assert abs(float(values[place, 0]) - float(logp[row, tokens[row]])) < 2e-5
        top_values, top_indices = torch.topk(logp[row], have)
        assert torch.allclose(values[place, 1 : 1 + have].double(), top_values, atol=2e-5, rtol=0)
        picked = indices[place, :have].tolist()
        assert len(set(picked)) == have
        assert torch.allclose(logp[row, picked], top_values, atol=1e-12, rtol=0)  # the same values, whatever the tie order
        assert all(i == -1 for i in indices[place, have:].tolist())
        assert all(math.isinf(v) and v < 0 for v in values[place, 1 + have :].tolist())
    if V > 300 and 0 in rows:
        assert indices[rows.index(0), :2].tolist() == [7, 300]
    # tokens given per report instead of per row
    per_report = torch.tensor([int(tokens[row]) for row in rows], dtype=torch.int32, device=DEV)
    again = torch.empty((len(rows), 1), device=DEV)
    kernels().logprob_report(
        logits.to(DEV), torch.tensor(rows, dtype=torch.int32, device=DEV), per_report, 0, again,
        torch.empty((len(rows), 0), dtype=torch.int32, device=DEV), tokens_by_row=False,
    )
    assert torch.equal(again.cpu()[:, 0], values[:, 0])


def _sample_both(logits, temperature, top_k, top_p, min_p, seeds):
    n, V = logits.shape
    t = lambda values, dtype: torch.tensor(values, dtype=dtype)
    args = (t(temperature, torch.float32), t(top_k, torch.int32), t(top_p, torch.float32), t(min_p, torch.float32), t(seeds, torch.int64))
    expected = torch.empty(n, dtype=torch.int32)
    ref.sample(logits, None, *args, expected)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    work = torch.empty(kernels().sample_work_floats(n, V), device=DEV)
    kernels().sample(logits.to(DEV), work, *(a.to(DEV) for a in args), out)
    return out.cpu().tolist(), expected.tolist()


@pytest.mark.parametrize("V", [331, 5000, 151936])
def test_sample_matches_the_reference_draws(V):
    from kairyu_b200.sampling.rng import as_signed64, mix_seed

    n = 24
    logits = rand(n, V, seed=42, scale=2.0)
    temperature = [0.8] * 6 + [1.0] * 6 + [0.0] * 2 + [1.7] * 10
    top_k = [-1, 5, 50, -1, 1, 20] * 4
    top_p = [1.0, 1.0, 0.9, 0.9, 0.5, 0.3] * 4
    min_p = [0.0, 0.0, 0.0, 0.05, 0.0, 0.2] * 4
    seeds = [as_signed64(mix_seed(1234 + r, r)) for r in range(n)]
    got, expected = _sample_both(logits, temperature, top_k, top_p, min_p, seeds)
    assert got == expected


def test_top_p_threshold_with_and_without_the_heavy_entries_reaching_it():
    """The top-p search looks at the entries of at least 1/65536 of the mass first.  Peaked rows (a few
    tokens carry the mass: those entries reach the target) and flat rows over a vocabulary of 151,936
    (no entry is that heavy, or too few: the search runs again over everything) give the reference's draws."""
    from kairyu_b200.sampling.rng import as_signed64, mix_seed

    V, n = 151936, 12
    g = torch.Generator().manual_seed(46)
    logits = torch.randn(n, V, generator=g)
    logits[0::3] *= 0.01                       # flat: every entry near 1 / V
    logits[1::3] *= 4.0                        # peaked
    logits[2::3] = logits[2::3] * 0.3          # flat, with a handful of heavy tokens that hold a third of the mass
    logits[2::3, :5] += 10.5
    top_p = [0.9, 0.9, 0.9, 0.5, 0.5, 0.5, 0.99, 0.99, 0.2, 0.05, 0.999, 0.7]
    seeds = [as_signed64(mix_seed(77 + r, r)) for r in range(n)]
    got, expected = _sample_both(logits, [1.0] * n, [-1] * n, top_p, [0.0] * n, seeds)
    assert got == expected


def test_sample_respects_the_filters_over_many_seeds():
    from kairyu_b200.sampling.rng import as_signed64, mix_seed

    V = 200
    base = torch.zeros(V)
    base[:4] = torch.log(torch.tensor([0.5, 0.25, 0.15, 0.1])) + 10.0
    base[4:] = -20.0
    n = 64
    logits = base.repeat(n, 1)
    seeds = [as_signed64(mix_seed(99, p)) for p in range(n)]
    got, expected = _sample_both(logits, [1.0] * n, [-1] * n, [0.7] * n, [0.0] * n, seeds)
    assert got == expected
    assert set(got) <= {0, 1}  # 0.5 + 0.25 reaches 0.7; the third token is cut
    assert len(set(got)) == 2
    got, _ = _sample_both(logits, [1.0] * n, [3] * n, [1.0] * n, [0.0] * n, seeds)
    assert set(got) == {0, 1, 2}


def test_sample_frequencies_follow_the_distribution():
    from kairyu_b200.sampling.rng import as_signed64, mix_seed

    V = 50
    probs = torch.tensor([0.4, 0.3, 0.2, 0.1] + [0.0] * (V - 4))
    logits = torch.log(probs.clamp(min=1e-30))
    n = 4000
    seeds = [as_signed64(mix_seed(7, p)) for p in range(n)]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    t = lambda values, dtype: torch.tensor(values, dtype=dtype, device=DEV)
    kernels().sample(
        logits.repeat(n, 1).to(DEV), torch.empty(kernels().sample_work_floats(n, V), device=DEV), t([1.0] * n, torch.float32), t([-1] * n, torch.int32),
        t([1.0] * n, torch.float32), t([0.0] * n, torch.float32), t(seeds, torch.int64), out,
    )
    counts = torch.bincount(out.cpu().long(), minlength=V).float() / n
    assert (counts[:4] - probs[:4]).abs().max() < 0.03
    assert counts[4:].sum() == 0


def test_sampling_kernels_draw_what_the_reference_sampler_drew():
    """tests/golden/sampler.pt: tokens the reference's own ``Sampler.sample`` drew for 56 cases of
    temperature, top-k, top-p, min-p, seeds, positions and penalties; the device pipeline (logit
    edits, radix-descent filters, Gumbel arg-max) draws the same tokens."""
    from pathlib import Path

    from kairyu_b200.sampling import Sampler
    from test_sampling_cpu import sampler_rows_of

    cases = torch.load(Path(__file__).resolve().parent / "golden" / "sampler.pt")
    for vocab, entries in sampler_rows_of(cases).items():
        sampler = Sampler(vocab, DEV)
        logits = torch.stack([entry[1] for entry in entries]).to(DEV)
        got = sampler.sample(logits, [entry[0] for entry in entries]).tolist()
        assert got == [entry[2] for entry in entries], vocab
