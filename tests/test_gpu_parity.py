"""Parity of the CUDA library (called through its C ABI via ctypes) with the CPU oracle and with
the golden vectors generated from the reference.  All tests need a GPU.

Error measure everywhere: rel_err(a, b) = the larger of max|a-b| / max|b| and mean|a-b| / mean|b|.
Tolerances: float32 1e-5; bfloat16 / float16 2e-2 (the oracle then runs in float32 on the
rounded inputs); integer tables bit-exact.
"""
import hashlib
import math

import numpy as np
import pytest
import torch

from oracle import hsa_oracle as orc
from tests.conftest import rel_err
from tests.test_oracle_golden import DIGESTS, WEIGHT_NAMES, config1_inputs

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


@pytest.fixture(scope="module")
def hsa():
    import sparseattention_b200 as pkg
    assert torch.cuda.is_available()
    return pkg


def dev(t):
    return t.cuda() if isinstance(t, torch.Tensor) else torch.from_numpy(np.asarray(t)).cuda()


# ------------------------------------------------------------------------------------ topology
def _digest(t):
    h = hashlib.sha256()
    h.update(t["forward_idx"].to(torch.int32).cpu().contiguous().numpy().tobytes())
    h.update(t["forward_mask"].to(torch.bool).cpu().contiguous().numpy().tobytes())
    h.update(t["backward_gather"].to(torch.int32).cpu().contiguous().numpy().tobytes())
    return h.hexdigest()[:32]


def test_topology_bit_exact(hsa, golden):
    g = golden("topology.npz")
    for N in (2, 4, 8, 16, 32):
        for c in (1, 0):
            t = hsa.build_tree_topology(N, is_causal=bool(c), device="cuda")
            tag = f"N{N}_c{c}"
            assert t["forward_idx"].dtype == torch.int32 and t["forward_mask"].dtype == torch.bool
            assert np.array_equal(t["forward_idx"].cpu().numpy(), g[f"idx_{tag}"])
            assert np.array_equal(t["forward_mask"].cpu().numpy(), g[f"mask_{tag}"])
            assert np.array_equal(t["backward_gather"].cpu().numpy(), g[f"gather_{tag}"])
    stored = {(int(n), int(c)): str(h) for n, c, h in zip(g["digest_N"], g["digest_causal"], g["digest_hex"])}
    stored.update(DIGESTS)
    for (N, c), hexd in stored.items():
        assert _digest(hsa.build_tree_topology(N, is_causal=bool(c), device="cuda")) == hexd, (N, c)
    # N = 1: no levels, a single row that gathers nothing
    t = hsa.build_tree_topology(1, True, device="cuda")
    assert t["forward_idx"].shape == (1, 0) and t["backward_gather"].tolist() == [[-1, -1, -1]]
    # against the oracle's explicit climb
    for N in (64, 1024):
        for c in (True, False):
            t = hsa.build_tree_topology(N, c, device="cuda")
            o = orc.build_tree_topology(N, c)
            for k in o:
                assert np.array_equal(t[k].cpu().numpy(), o[k])
    # unmasked entries under causal masking: exactly half
    t = hsa.build_tree_topology(4096, True, device="cuda")
    assert int((~t["forward_mask"]).sum()) == 24576


# ------------------------------------------------------------------------- generate_span_input_Y
def test_span_input_y_golden_bit_exact(hsa, golden):
    g = golden("span_input_y.npz")
    for name in "abcd":
        y = hsa.generate_span_input_Y(dev(g[f"x_{name}"]))
        assert np.array_equal(y.cpu().numpy(), g[f"y_{name}"]), name
    y = hsa.generate_span_input_Y(dev(g["x_bf16"]).to(torch.bfloat16))
    assert np.array_equal(y.float().cpu().numpy(), g["y_bf16"])
    assert hsa.generate_span_input_Y(torch.zeros(1, 1, 4, device="cuda")) is None


@pytest.mark.parametrize("shape", [(2, 16, 8), (1, 12, 5), (2, 1000, 24), (1, 4096, 512), (3, 37, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_span_input_y_forward_backward(hsa, shape, dtype):
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(*shape, generator=gen).to(dtype)
    xo = x.detach().clone().requires_grad_()
    yo = orc.generate_span_input_Y(xo)
    gy = torch.randn(yo.shape, generator=gen).to(dtype)
    yo.backward(gy)
    xc = x.detach().cuda().requires_grad_()
    yc = hsa.generate_span_input_Y(xc)
    assert torch.equal(yc.detach().cpu(), yo.detach())           # bit-exact forward
    yc.backward(gy.cuda())
    assert rel_err(xc.grad.float().cpu(), xo.grad.float()) <= (1e-6 if dtype == torch.float32 else 1e-2)
    # non-contiguous input (a slice of a wider tensor)
    wide = torch.randn(shape[0], shape[1], shape[2] + 8, generator=gen).to(dtype).cuda()
    yv = hsa.generate_span_input_Y(wide[:, :, :shape[2]])
    assert torch.equal(yv, hsa.generate_span_input_Y(wide[:, :, :shape[2]].contiguous()))


# ------------------------------------------------------------------------------- parent nodes
def test_parent_nodes_triton_golden(hsa, golden):
    g = golden("triton_ops.npz")
    names = ("Qp", "Kp", "Vp", "Kc", "Vc")
    ts = [dev(g[f"parent.{n}"]).requires_grad_() for n in names]
    o = hsa.build_parent_nodes(*ts)
    o.backward(dev(g["parent.go"]))
    assert rel_err(o.detach().cpu(), g["parent.out"]) < 1e-5
    for n, t in zip(names, ts):
        assert rel_err(t.grad.cpu(), g[f"parent.d{n}"]) < 1e-5, n


@pytest.mark.parametrize("B,P,H,D", [(1, 1, 1, 8), (2, 8, 3, 16), (2, 33, 5, 24), (1, 256, 8, 64), (2, 64, 16, 128),
                                     (1, 5, 2, 10), (1, 7, 1, 256), (1, 3, 2, 200)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_parent_nodes_vs_oracle(hsa, B, P, H, D, dtype):
    gen = torch.Generator().manual_seed(B * 1000 + P)
    shapes = [(B, P, H, D)] * 3 + [(B, 2 * P, H, D)] * 2
    ins = [torch.randn(*s, generator=gen).to(dtype) for s in shapes]
    go = torch.randn(B, P, H, D, generator=gen).to(dtype)
    ref_in = [t.detach().float().clone().requires_grad_() for t in ins]
    ro = orc.build_parent_nodes(*ref_in)
    ro.backward(go.float())
    cu_in = [t.detach().cuda().requires_grad_() for t in ins]
    co = hsa.build_parent_nodes(*cu_in)
    assert co.dtype == dtype and co.shape == (B, P, H, D)
    co.backward(go.cuda())
    tol = TOL[dtype]
    assert rel_err(co.detach().float().cpu(), ro.detach()) < tol
    for c, r in zip(cu_in, ref_in):
        assert rel_err(c.grad.float().cpu(), r.grad) < tol


def test_parent_nodes_split_views_no_copy(hsa):
    """Level slices of one [B, N-1, H, D] projection (torch.split views) are taken as they are."""
    gen = torch.Generator().manual_seed(5)
    B, N, H, D = 2, 32, 4, 32
    allq, allk, allv = (torch.randn(B, N - 1, H, D, generator=gen).cuda() for _ in range(3))
    kc, vc = (torch.randn(B, N, H, D, generator=gen).cuda() for _ in range(2))
    sizes = [16, 8, 4, 2, 1]
    q0, k0, v0 = (torch.split(t, sizes, dim=1)[0] for t in (allq, allk, allv))
    assert not q0.is_contiguous()
    o = hsa.build_parent_nodes(q0, k0, v0, kc, vc)
    r = orc.build_parent_nodes(q0.cpu(), k0.cpu(), v0.cpu(), kc.cpu(), vc.cpu())
    assert rel_err(o.cpu(), r) < 1e-5


# ------------------------------------------------------------------------------ span attention
def test_span_attention_triton_golden(hsa, golden):
    g = golden("triton_ops.npz")
    for tag in ("span_a", "span_b", "span_r0"):
        B, N, H, D, R = (int(v) for v in g[f"{tag}.meta"])
        for c in (1, 0):
            t = hsa.build_tree_topology(N, bool(c), device="cuda")
            q, k, v = (dev(g[f"{tag}.{n}"]).requires_grad_() for n in "QKV")
            o = hsa.hierarchical_attention(q, k, v, t["forward_idx"], t["backward_gather"],
                                           t["forward_mask"] if c else None, R)
            o.backward(dev(g[f"{tag}.go"]))
            assert rel_err(o.detach().cpu(), g[f"{tag}.out_c{c}"]) < 1e-5, (tag, c)
            assert rel_err(q.grad.cpu(), g[f"{tag}.dQ_c{c}"]) < 1e-5, (tag, c)
            assert rel_err(k.grad.cpu(), g[f"{tag}.dK_c{c}"]) < 1e-5, (tag, c)
            assert rel_err(v.grad.cpu(), g[f"{tag}.dV_c{c}"]) < 1e-5, (tag, c)


SPAN_CASES = [
    # B, N, H, D, R
    (1, 1, 1, 8, 2), (1, 2, 2, 8, 0), (2, 4, 1, 16, 1), (1, 8, 3, 16, 3), (2, 16, 3, 24, 2), (1, 64, 2, 32, 5),
    (1, 64, 4, 64, 100), (1, 128, 2, 128, 16), (2, 256, 3, 64, 8), (1, 512, 2, 10, 4), (1, 2048, 1, 64, 16),
    (1, 32, 1, 256, 3), (1, 16, 2, 200, 2),
]


def run_span_case(hsa, B, N, H, D, R, causal, dtype, algo=0, seed=0, check_grad=True):
    from sparseattention_b200.ops import functional as F
    gen = torch.Generator().manual_seed(seed + N * 7 + R)
    Q = torch.randn(B, N, H, D, generator=gen).to(dtype)
    K = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    V = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    go = torch.randn(B, N, H, D, generator=gen).to(dtype)
    q, k, v = (t.detach().float().clone().requires_grad_() for t in (Q, K, V))
    ro, rlse = orc.hierarchical_attention(q, k, v, R, causal, return_lse=True)
    Qc, Kc, Vc = Q.cuda(), K.cuda(), V.cuda()
    out, lse = F.span_attention_forward(Qc, Kc, Vc, R, causal, need_lse=True, algo=algo)
    tol = TOL[dtype]
    assert out.dtype == dtype
    assert rel_err(out.float().cpu(), ro.detach()) < tol
    assert rel_err(lse.cpu(), rlse.detach()) < (1e-5 if dtype == torch.float32 else 1e-4)
    if not check_grad:
        return
    ro.backward(go.float())
    try:
        dq, dk, dv = F.span_attention_backward(Qc, Kc, Vc, out, lse, go.cuda(), R, causal, algo=algo)
    except Exception as exc:   # a window too wide for the backward's shared memory: the automatic choice takes over
        if algo != 2 or "fits shared memory" not in str(exc):
            raise
        algo = 0
        dq, dk, dv = F.span_attention_backward(Qc, Kc, Vc, out, lse, go.cuda(), R, causal, algo=algo)
    assert rel_err(dq.float().cpu(), q.grad) < tol
    assert rel_err(dk.float().cpu(), k.grad) < tol
    assert rel_err(dv.float().cpu(), v.grad) < tol
    # rows nobody attends to (root; right children when causal) must be exact zeros
    if N > 1:
        assert float(dk[:, 2 * N - 2].abs().max()) == 0.0 and float(dv[:, 2 * N - 2].abs().max()) == 0.0
    dq2, dk2, dv2 = F.span_attention_backward(Qc, Kc, Vc, out, lse, go.cuda(), R, causal, algo=algo)
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2) and torch.equal(dq, dq2)   # deterministic


@pytest.mark.parametrize("case", SPAN_CASES)
@pytest.mark.parametrize("causal", [True, False])
def test_span_attention_fp32_vs_oracle(hsa, case, causal):
    run_span_case(hsa, *case, causal, torch.float32, algo=1)


@pytest.mark.parametrize("case", [(2, 16, 3, 24, 2), (1, 128, 2, 128, 16), (2, 256, 3, 64, 8), (1, 64, 2, 32, 5)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_span_attention_half_vs_oracle_portable(hsa, case, causal, dtype):
    run_span_case(hsa, *case, causal, dtype, algo=1)


TC_CASES = [(1, 64, 1, 64, 0), (2, 64, 3, 64, 5), (1, 128, 2, 128, 16), (2, 256, 3, 64, 8), (1, 512, 2, 128, 33),
            (1, 1024, 1, 64, 16), (1, 4096, 2, 128, 16), (1, 2048, 1, 128, 60), (1, 256, 2, 64, 300),
            (1, 16384, 1, 64, 16), (1, 65536, 1, 64, 1)]


@pytest.mark.parametrize("case", [(2, 64, 3, 64, 0), (1, 64, 1, 64, 16), (2, 512, 4, 64, 16), (1, 128, 2, 64, 1), (1, 1024, 5, 64, 40),
                                  (1, 32, 2, 128, 3), (2, 256, 3, 128, 16), (1, 4096, 2, 128, 16), (1, 8192, 1, 64, 7),
                                  (1, 2048, 2, 128, 33)])
@pytest.mark.parametrize("causal", [True, False])
def test_span_attention_fp32_staged_forward(hsa, case, causal):
    """float32 with head dim 64 / 128: the automatic choice stages a tile's rows in shared memory (forward); same bound
    as the portable kernel, which stays the backward and the fallback."""
    run_span_case(hsa, *case, causal, torch.float32, algo=0)


@pytest.mark.parametrize("case", TC_CASES)
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_span_attention_tensor_core(hsa, case, causal, dtype):
    """The tensor-core forward and backward (algo 2) against the oracle."""
    run_span_case(hsa, *case, causal, dtype, algo=2)


@pytest.mark.parametrize("case", [(1, 128, 1, 64, 0), (2, 128, 3, 64, 5), (1, 256, 2, 128, 16), (2, 1024, 3, 64, 8),
                                  (1, 4096, 2, 128, 16), (1, 8192, 1, 128, 7), (3, 512, 5, 128, 1),
                                  (1, 16384, 1, 128, 16), (1, 32768, 1, 64, 9)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_span_attention_tensor_core_128_leaf_tiles(hsa, case, dtype):
    """The 128-leaf-tile forward (algo 4, causal) against the oracle, and bit-for-bit LSE agreement is not
    required between tile sizes, only the common tolerance."""
    run_span_case(hsa, *case, True, dtype, algo=4)          # 128-leaf forward and the 8-warp backward
    run_span_case(hsa, *case, True, dtype, algo=3)          # 64-leaf forward and the 4-warp backward


@pytest.mark.parametrize("case", [(1, 128, 2, 128, 17), (2, 256, 3, 128, 32), (1, 1024, 2, 64, 32), (1, 4096, 2, 128, 24),
                                  (1, 8192, 1, 128, 32), (1, 16384, 1, 128, 32), (1, 32768, 1, 64, 31)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_span_attention_128_leaf_tiles_wide_window(hsa, case, dtype):
    """The 128-leaf-tile forward with a halo of two 16-leaf blocks (radius 17..32): 256-byte rows load the second half of
    V over the dead K plane; beyond N = 8192 a warp scores five key blocks."""
    run_span_case(hsa, *case, True, dtype, algo=4, check_grad=False)


@pytest.mark.parametrize("case", [(2, 256, 12, 64, 8), (1, 1024, 12, 64, 16), (1, 2048, 12, 128, 16),
                                  (1, 4096, 16, 128, 16)])
@pytest.mark.parametrize("algo", [0, 3])
def test_span_attention_tensor_core_12_and_16_heads(hsa, case, algo):
    """Forward and backward at the head counts the reference's models use (12) and at the benchmarked layer
    shape (16 heads of 128, N=4096): automatic choice (128-leaf forward, 8-warp backward) and the 64-leaf /
    4-warp kernels."""
    run_span_case(hsa, *case, True, torch.bfloat16, algo=algo)


def test_tensor_core_kernel_refuses_what_it_cannot_take(hsa):
    from sparseattention_b200._lib import HsaError
    from sparseattention_b200.ops import functional as F
    q = torch.randn(1, 32, 1, 64, device="cuda", dtype=torch.bfloat16)          # N < 64
    kv = torch.randn(1, 63, 1, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(HsaError):
        F.span_attention_forward(q, kv, kv, 4, True, algo=2)
    q = torch.randn(1, 64, 1, 64, device="cuda")                                 # float32
    kv = torch.randn(1, 127, 1, 64, device="cuda")
    with pytest.raises(HsaError):
        F.span_attention_forward(q, kv, kv, 4, True, algo=2)
    F.span_attention_forward(q, kv, kv, 4, True, algo=0)                          # automatic choice still works
    qb = torch.randn(1, 128, 1, 64, device="cuda", dtype=torch.bfloat16)
    kvb = torch.randn(1, 255, 1, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(HsaError):
        F.span_attention_forward(qb, kvb, kvb, 33, True, algo=4)                 # radius beyond the 128-leaf kernel
    with pytest.raises(HsaError):
        F.span_attention_forward(qb, kvb, kvb, 4, False, algo=4)                 # not causal


def test_span_attention_rejects_foreign_tables(hsa):
    from sparseattention_b200._lib import HsaError
    N = 16
    t = hsa.build_tree_topology(N, True, device="cuda")
    bad = t["forward_idx"].clone()
    bad[3, 1] += 1
    q = torch.randn(1, N, 1, 16, device="cuda")
    kv = torch.randn(1, 2 * N - 1, 1, 16, device="cuda")
    with pytest.raises(HsaError):
        hsa.hierarchical_attention(q, kv, kv, bad, t["backward_gather"], t["forward_mask"], 2)


def test_span_attention_b16_h8_n512_bf16_forward_backward(hsa):
    """B16 H8 N512 Dh64, causal window 8, bf16, upstream gradient ~ N(0,1)."""
    run_span_case(hsa, 16, 512, 8, 64, 8, True, torch.bfloat16, algo=0, seed=2)


@pytest.mark.parametrize("case", [(1, 64, 1, 64, 16), (2, 64, 3, 128, 3), (1, 128, 2, 128, 16), (2, 2048, 2, 64, 0),
                                  (1, 16384, 2, 64, 16), (1, 32768, 1, 128, 11)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_span_attention_automatic_choice_causal(hsa, case, dtype):
    """algo 0 on causal half-precision inputs with a window of at most 16: the backward runs the 8-warp
    task-parallel kernel (single-tile tree N=64, one and two tree blocks per query block)."""
    run_span_case(hsa, *case, True, dtype, algo=0)


def test_span_attention_full_size_properties(hsa):
    """The benchmarked layer shape (N=4096, H16, Dh128, bf16): size-independent properties.

    (1) rows of a softmax average: with V == 1 everywhere the output is exactly 1;
    (2) linearity in V: out(V1 + V2) == out(V1) + out(V2) up to bf16 rounding;
    (3) causality: changing K/V of leaves >= n0 leaves outputs of leaves < n0 untouched, bit for bit;
    (4) a random sample of leaves agrees with the oracle evaluated on just those leaves.
    """
    from sparseattention_b200.ops import functional as F
    B, N, H, D, R = 2, 4096, 16, 128, 16
    gen = torch.Generator().manual_seed(9)
    Q = torch.randn(B, N, H, D, generator=gen).bfloat16().cuda()
    K = torch.randn(B, 2 * N - 1, H, D, generator=gen).bfloat16().cuda()
    V = torch.randn(B, 2 * N - 1, H, D, generator=gen).bfloat16().cuda()
    out, lse = F.span_attention_forward(Q, K, V, R, True)
    ones, _ = F.span_attention_forward(Q, K, torch.ones_like(V), R, True)
    assert float((ones.float() - 1).abs().max()) < 1e-2
    V2 = torch.randn(B, 2 * N - 1, H, D, generator=gen).bfloat16().cuda()
    o2, _ = F.span_attention_forward(Q, K, V2, R, True)
    o12, _ = F.span_attention_forward(Q, K, (V.float() + V2.float()).bfloat16(), R, True)
    assert rel_err(o12.float().cpu(), (out.float() + o2.float()).cpu()) < 3e-2
    n0 = 1000
    K3, V3 = K.clone(), V.clone()
    K3[:, n0:N] += 1.0
    V3[:, n0:N] -= 1.0
    o3, _ = F.span_attention_forward(Q, K3, V3, R, True)
    assert torch.equal(o3[:, :n0], out[:, :n0])
    # sampled leaves against the oracle
    rows, valid = orc.span_candidates(N, R, True)
    sample = torch.tensor([0, 1, 2, 17, 255, 256, 1023, 2048, 3000, 4095])
    q = Q[:, sample].float().cpu()
    k = K.float().cpu()[:, rows[sample]]
    v = V.float().cpu()[:, rows[sample]]
    logits = torch.einsum("bnhd,bnchd->bnhc", q, k) / math.sqrt(D)
    logits = logits.masked_fill(~valid[sample][None, :, None, :], float("-inf"))
    w = torch.softmax(logits, dim=-1)
    want = torch.einsum("bnhc,bnchd->bnhd", w, v)
    assert rel_err(out[:, sample].float().cpu(), want) < 2e-2
    assert rel_err(lse[:, sample].cpu(), torch.logsumexp(logits, dim=-1)) < 1e-4


# ------------------------------------------------------------------------------------- tcgen05 products
GEMM_CASES = [
    # batches, rows, N, K
    (1, 128, 256, 64), (1, 128, 128, 64), (1, 256, 512, 512), (1, 100, 256, 72), (2, 200, 520, 136), (3, 64, 64, 512),
    (1, 1000, 1536, 512), (1, 384, 50304, 512), (4, 33, 1024, 2048), (1, 4096, 512, 2048), (1, 8, 8, 8),
]


@pytest.mark.parametrize("shape", [(3, 8), (1000, 512), (4, 300, 2048), (32768, 512), (257, 50304)])
def test_column_sums(hsa, shape):
    from sparseattention_b200.ops.gemm import column_sums
    gen = torch.Generator().manual_seed(shape[-1])
    x = torch.randn(*shape, generator=gen).bfloat16()
    want = x.double().reshape(-1, shape[-1]).sum(dim=0)
    got = column_sums(x.cuda())
    assert got.dtype == torch.float32 and rel_err(got.cpu(), want) < 1e-5
    assert torch.equal(got, column_sums(x.cuda()))               # fixed summation order


@pytest.mark.parametrize("shape", [(5, 8), (2, 333, 512), (8, 4095, 512), (1000, 2048)])
@pytest.mark.parametrize("sites", [None, (3, 0), (4, 9)])
def test_masked_cast_with_column_sums(hsa, shape, sites):
    """One pass = dropout mask (that of DropoutSpec.apply on the same logical tensor) * float32 -> bfloat16, plus the column
    sums of what was written."""
    from sparseattention_b200.ops.gemm import DropoutSpec, column_sums, masked_cast_with_sums
    gen = torch.Generator().manual_seed(shape[-1] + len(shape))
    x = torch.randn(*shape, generator=gen).cuda()
    key = torch.tensor([987654321], dtype=torch.int64, device="cuda")
    spec = None if sites is None else DropoutSpec(key, 0.1, *sites)
    got, sums = masked_cast_with_sums(x, spec)
    x3 = x.reshape(1, -1, shape[-1])
    if spec is None:
        want = x.bfloat16()
    else:
        want = spec.apply(x3, torch.empty_like(x3, dtype=torch.bfloat16), 0, shape[-1], shape[-1], x3.size(1)).reshape(shape)
    assert torch.equal(got, want)
    want_sums = got.double().reshape(-1, shape[-1]).sum(dim=0)
    assert rel_err(sums.cpu(), want_sums.cpu()) < 1e-5
    if spec is not None and got.numel() >= 100000:
        dropped = float((got == 0).float().mean())
        assert abs(dropped - (0.1 if sites[1] == 0 else 0.19)) < 0.01


def _gemm_inputs(batches, rows, N, K, seed):
    gen = torch.Generator().manual_seed(seed)
    A = torch.randn(batches, rows, K, generator=gen).bfloat16()
    W = torch.randn(N, K, generator=gen).bfloat16()
    bias = torch.randn(N, generator=gen)
    return A, W, bias


@pytest.mark.parametrize("case", GEMM_CASES)
def test_gemm_forward_product(hsa, case):
    """C = A W^T (+ bias) on the tcgen05 kernel against a float64 product of the same bf16 operands."""
    from sparseattention_b200.ops.gemm import gemm, gemm_aborts
    batches, rows, N, K = case
    A, W, bias = _gemm_inputs(*case, seed=rows + N)
    want = torch.einsum("brk,nk->brn", A.double(), W.double())
    got = gemm(A.cuda(), W.cuda(), out_dtype=torch.float32)
    assert rel_err(got.cpu(), want) < 1e-5
    got = gemm(A.cuda(), W.cuda(), bias=bias.cuda())
    assert got.dtype == torch.bfloat16 and rel_err(got.float().cpu(), want + bias.double()) < 1e-2
    # operands and result as strided views of wider tensors; a forced split along K
    wideA = torch.zeros(batches, rows + 3, K + 16, dtype=torch.bfloat16, device="cuda")
    wideA[:, 1:rows + 1, 8:K + 8] = A.cuda()
    wideC = torch.full((batches, rows, N + 24), 7.0, dtype=torch.float32, device="cuda")
    gemm(wideA[:, 1:rows + 1, 8:K + 8], W.cuda(), out=wideC[:, :, 8:N + 8], splits=2 if K >= 128 else 1)
    assert rel_err(wideC[:, :, 8:N + 8].cpu(), want) < 1e-5
    assert float((wideC[:, :, :8] - 7).abs().max()) == 0 and float((wideC[:, :, N + 8:] - 7).abs().max()) == 0
    assert gemm_aborts() == 0


@pytest.mark.parametrize("case", GEMM_CASES)
def test_gemm_transposed_operands(hsa, case):
    """The two backward products of a linear layer: dX = dY W (B read as [K, N]) and dW = dY^T X summed over all batch
    entries (both operands read transposed), with automatic and forced split-K; accumulation into float32."""
    from sparseattention_b200.ops.gemm import gemm, gemm_aborts
    batches, rows, N, K = case
    A, W, _ = _gemm_inputs(*case, seed=rows * 3 + K)
    gen = torch.Generator().manual_seed(N)
    dY = torch.randn(batches, rows, N, generator=gen).bfloat16()
    want_dx = torch.einsum("brn,nk->brk", dY.double(), W.double())
    got = gemm(dY.cuda(), W.cuda(), b_t=True, out_dtype=torch.float32)
    assert rel_err(got.cpu(), want_dx) < 1e-5
    if K % 8 == 0:
        want_dw = torch.einsum("brn,brk->nk", dY.double(), A.double())
        for splits in (None, 1, 3):
            got = gemm(dY.cuda(), A.cuda(), a_t=True, b_t=True, out_dtype=torch.float32, splits=splits)
            assert got.shape == (N, K) and rel_err(got.cpu(), want_dw) < 1e-5, splits
        acc = torch.ones(N, K, device="cuda")
        gemm(dY.cuda(), A.cuda(), a_t=True, b_t=True, out=acc, accumulate=True)
        assert rel_err(acc.cpu(), want_dw + 1) < 1e-5
    assert gemm_aborts() == 0


def test_linear_matches_torch(hsa):
    """ops.gemm.linear against F.linear in float64 on the bf16-rounded operands: output and the three gradients."""
    from sparseattention_b200.ops.gemm import linear
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(4, 300, 512, generator=gen).bfloat16()
    w = torch.randn(1024, 512, generator=gen) * 0.05
    b = torch.randn(1024, generator=gen)
    gy = torch.randn(4, 300, 1024, generator=gen).bfloat16()
    xr, wr, br = x.double().requires_grad_(), w.bfloat16().double().requires_grad_(), b.double().requires_grad_()
    torch.nn.functional.linear(xr, wr, br).backward(gy.double())
    xc, wc, bc = x.cuda().requires_grad_(), w.cuda().requires_grad_(), b.cuda().requires_grad_()
    y = linear(xc, wc, bc)
    y.backward(gy.cuda())
    assert y.dtype == torch.bfloat16 and rel_err(y.detach().float().cpu(), torch.nn.functional.linear(xr, wr, br).detach()) < 1e-2
    assert xc.grad.dtype == torch.bfloat16 and rel_err(xc.grad.float().cpu(), xr.grad) < 1e-2
    assert wc.grad.dtype == torch.float32 and rel_err(wc.grad.cpu(), wr.grad) < 1e-4
    assert rel_err(bc.grad.cpu(), br.grad) < 1e-4


def test_gemm_fused_tails(hsa):
    """The element-wise tails of hsa_gemm_ex against the same steps done by hand: bias + relu, residual, bfloat16 copy,
    gate; and dropout inside the epilogue against the plain product followed by hsa_dropout_apply (which must
    regenerate exactly the same masks: that is what the backward relies on)."""
    from sparseattention_b200.ops.gemm import DropoutSpec, gemm
    gen = torch.Generator().manual_seed(5)
    B, rows, N, K = 2, 300, 512, 256
    A = torch.randn(B, rows, K, generator=gen).bfloat16().cuda()
    W = (torch.randn(N, K, generator=gen) * 0.1).bfloat16().cuda()
    bias = torch.randn(N, generator=gen).cuda()
    res = torch.randn(B, rows, N, generator=gen).cuda()
    plain = gemm(A, W, out_dtype=torch.float32)
    got = gemm(A, W, bias=bias, relu=True, out_dtype=torch.float32)
    assert rel_err(got.cpu(), torch.relu(plain + bias).cpu()) < 1e-6
    copy = torch.empty(B, rows, N, dtype=torch.bfloat16, device="cuda")
    got = gemm(A, W, bias=bias, out=torch.empty_like(res), residual=res, copy_bf16=copy)
    assert rel_err(got.cpu(), (plain + bias + res).cpu()) < 1e-6 and torch.equal(copy, got.bfloat16())
    gate = torch.randn(B, rows, N, generator=gen).bfloat16().cuda()
    got = gemm(A, W, out_dtype=torch.float32, gate=gate, gate_scale=1.25)
    assert rel_err(got.cpu(), torch.where(gate > 0, plain * 1.25, torch.zeros_like(plain)).cpu()) < 1e-6
    # dropout: epilogue == product, then apply; one and two masks, a column range, rows of a larger logical tensor
    key = torch.tensor([1234567], dtype=torch.int64, device="cuda")
    for site1 in (0, 9):
        spec = DropoutSpec(key, 0.1, 3, site1)
        want = gemm(A, W)
        spec.apply(want, want, 256, 256, N, 1000, 17)
        got = gemm(A, W, dropout=spec, drop_cols=(256, 512), drop_rows_total=1000, drop_row_offset=17)
        assert torch.equal(got == 0, want == 0)                   # the same elements are dropped ...
        assert rel_err(got.float().cpu(), want.float().cpu()) < 1e-2   # ... and the kept ones agree up to one more bf16 rounding
        kept = float((got[..., 256:] != 0).float().mean())
        assert abs(kept - (0.9 ** (2 if site1 else 1))) < 0.01
        assert torch.equal(got[..., :256], gemm(A, W)[..., :256])
        ratio = got[..., 256:].float() / gemm(A, W)[..., 256:].float()
        scale = 1 / 0.9 ** (2 if site1 else 1)
        assert float((ratio[got[..., 256:] != 0] - scale).abs().max()) < 0.02
    # another key gives another mask; float32 input converts on the way; shifted columns
    spec = DropoutSpec(key, 0.1, 3)
    a = spec.apply(plain, torch.empty_like(plain, dtype=torch.bfloat16), 0, N, N, rows)
    b2 = DropoutSpec(key + 1, 0.1, 3).apply(plain, torch.empty_like(plain, dtype=torch.bfloat16), 0, N, N, rows)
    assert not torch.equal(a, b2)
    wide = torch.zeros(B, rows, 2 * N, dtype=torch.bfloat16, device="cuda")
    wide[..., N:] = plain.bfloat16()
    spec.apply(wide, wide, N, N, N, rows, 0, -N)
    assert torch.equal(wide[..., N:] == 0, a == 0) and rel_err(wide[..., N:].float().cpu(), a.float().cpu()) < 1e-2


@pytest.mark.parametrize("shape", [(2, 256, 256, 4, 512), (1, 1024, 512, 8, 2048), (3, 128, 128, 2, 256)])
def test_fused_decoder_layer_against_eager(hsa, shape):
    """The one-node decoder layer (tcgen05 products, fused tails, hand-written backward) under bf16 autocast: both
    outputs, both input gradients and every parameter gradient, no dropout.  The yardstick is the eager layer in
    float32 (Linear weights rounded to bfloat16, as autocast rounds them); the bound for each tensor is 2e-2, or,
    where bfloat16 itself costs more than that (the relu gate of the feed-forward flips for pre-activations near
    zero, which moves fc1's and norm2's gradients by several percent in ANY bf16 run), 1.25 x the error of the
    eager bf16-autocast layer on the same inputs."""
    import copy
    from sparseattention_b200.fused_layer import fused_layer_supported
    from sparseattention_b200.lm import DecoderLayer
    torch.backends.cuda.matmul.allow_tf32 = False
    B, N, d, H, ff = shape
    torch.manual_seed(N + d)
    layer = DecoderLayer(d, H, ff, dropout=0.0, window_size=16).cuda().train()
    with torch.no_grad():
        for prm in layer.parameters():                       # biases and norm parameters away from their trivial values
            if prm.dim() == 1:
                prm.add_(torch.randn_like(prm) * 0.1)
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(B, N, d, generator=gen).cuda()
    y = torch.randn(B, N - 1, d, generator=gen).cuda()
    gx = torch.randn(B, N, d, generator=gen).cuda()
    gy = torch.randn(B, N - 1, d, generator=gen).cuda()
    ref = copy.deepcopy(layer).float()
    ref.fused = False
    with torch.no_grad():
        for mod in ref.modules():
            if isinstance(mod, torch.nn.Linear):
                mod.weight.copy_(mod.weight.bfloat16().float())
    flag = torch.ones(1, device="cuda")

    def run(mod, autocast):
        for prm in mod.parameters():
            prm.grad = None
        xr, yr = x.clone().requires_grad_(), y.clone().requires_grad_()
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            if autocast and mod.fused:
                assert fused_layer_supported(mod, xr, yr, flag)
            xo, yo = mod(xr, yr, mask=flag)
        ((xo * gx).sum() + (yo * gy).sum()).backward()
        out = {"x_out": xo.detach(), "y_out": yo.detach(), "dx": xr.grad, "dy": yr.grad}
        for name, prm in mod.named_parameters():
            assert prm.grad is not None, name
            out[name] = prm.grad.clone()
        return {k: v.float().cpu() for k, v in out.items()}

    want = run(ref, False)
    layer.fused = True
    fused = run(layer, True)
    layer.fused = False
    eager = run(layer, True)
    assert fused["x_out"].dtype == torch.float32
    for name in want:
        bound = max(2e-2, 1.25 * rel_err(eager[name], want[name]))
        assert rel_err(fused[name], want[name]) < bound, name


@pytest.mark.parametrize("shape", [(2, 256, 256, 4, 512), (1, 2048, 512, 8, 512), (2, 512, 512, 4, 256)])
@pytest.mark.parametrize("p", [0.0, 0.1])
def test_parent_tree_launch_matches_per_level(hsa, shape, p):
    """One cooperative launch per tree (from level 1, and from level 3) against the launch-per-level path of the fused
    layer, same dropout key: outputs and all gradients agree to bfloat16 accuracy (the two paths round a few values
    differently in the last bit, which the relu gate of the feed-forward can amplify to a few percent in single entries
    of fc1's gradient; hence 5e-2 on the maximum and 1e-2 on the mean measure)."""
    import sparseattention_b200.fused_layer as fl
    from sparseattention_b200.lm import DecoderLayer
    B, N, d, H, ff = shape
    torch.manual_seed(N)
    layer = DecoderLayer(d, H, ff, dropout=p, window_size=16).cuda().train()
    x = torch.randn(B, N, d, device="cuda")
    y = torch.randn(B, N - 1, d, device="cuda")
    gx, gy = torch.randn_like(x), torch.randn_like(y)
    cfg = {"heads": H, "window": 16, "causal": True, "p": p, "eps": 1e-5}
    key = torch.tensor([4242], dtype=torch.int64, device="cuda")
    prm = list(fl.fused_layer_parameters(layer))
    results = {}
    old = fl.TREE_START_LEVEL
    try:
        for start in (None, 1, 3):
            fl.TREE_START_LEVEL = start
            for q in prm:
                q.grad = None
            xg, yg = x.clone().requires_grad_(), y.clone().requires_grad_()
            xo, yo = fl.FusedDecoderLayerFunction.apply(xg, yg, cfg, key, *prm)
            ((xo * gx).sum() + (yo * gy).sum()).backward()
            results[start] = [xo.detach(), yo.detach(), xg.grad, yg.grad] + [q.grad.clone() for q in prm]
    finally:
        fl.TREE_START_LEVEL = old
    from tests.conftest import max_rel_err, mean_rel_err
    relu_gated = {4 + 14, 4 + 15, 4 + 16, 4 + 17}   # norm2's and fc1's parameters: entries move with every flipped relu gate
    for start in (1, 3):
        for i, (got, want) in enumerate(zip(results[start], results[None])):
            assert max_rel_err(got.float().cpu(), want.float().cpu()) < (0.25 if i in relu_gated else 5e-2), (start, i)
            assert mean_rel_err(got.float().cpu(), want.float().cpu()) < 2e-2, (start, i)


def test_parent_tree_bounded_barrier(hsa):
    """The grid barrier of the tree launch gives up instead of hanging: with the test hook the barrier waits for one
    arrival more than there are thread blocks and for about a millisecond only; every block must leave, the status word
    must say so, and the next launch (hook off) must complete normally."""
    import sparseattention_b200.fused_layer as fl
    from sparseattention_b200 import _lib
    lib = _lib.load()
    B, N, d, H = 1, 256, 256, 4
    gen = torch.Generator(device="cuda").manual_seed(1)
    QKVp = torch.randn(B, N - 1, 3 * d, generator=gen, device="cuda").bfloat16()
    Rb = torch.randn(B, N - 1, d, generator=gen, device="cuda").bfloat16()
    KVc = torch.zeros(B, N - 1, 2 * d, device="cuda", dtype=torch.bfloat16)
    W = (torch.randn(2 * d, d, generator=gen, device="cuda") * 0.05).bfloat16()
    try:
        _lib.check(lib.hsa_debug_wait_test(2_000_000, 1), "hsa_debug_wait_test")
        state = fl._parent_tree_fwd(QKVp, Rb.clone(), KVc, W, N, H, 1, None)
        assert fl.parent_tree_status(state) == 1
    finally:
        _lib.check(lib.hsa_debug_wait_test(2_000_000_000, 0), "hsa_debug_wait_test")
    R2 = Rb.clone()
    state = fl._parent_tree_fwd(QKVp, R2, KVc, W, N, H, 1, None)
    assert fl.parent_tree_status(state) == 0
    assert bool(torch.isfinite(R2.float()).all()) and not torch.equal(R2[:, N // 2:], Rb[:, N // 2:])


def test_fused_decoder_layer_dropout(hsa):
    """With dropout the fused layer draws a new mask per call, yet forward and backward of one call agree on it: the
    layer is linear in the feed-forward output bias, so the gradient of sum(x_out) for that bias must equal the
    per-column sum of the kept-and-scaled mask, which the forward exposes as x_out(b2 + 1) - x_out(b2)."""
    from sparseattention_b200.lm import DecoderLayer
    torch.manual_seed(1)
    B, N, d, H, ff = 2, 256, 256, 4, 512
    layer = DecoderLayer(d, H, ff, dropout=0.1, window_size=16).cuda().train()
    x = torch.randn(B, N, d, device="cuda")
    y = torch.randn(B, N - 1, d, device="cuda")
    flag = torch.ones(1, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        a, _ = layer(x, y, mask=flag)
        b2, _ = layer(x, y, mask=flag)
    assert bool(torch.isfinite(a).all()) and not torch.equal(a, b2)
    layer.eval()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        e1, _ = layer(x, y, mask=flag)
        e2, _ = layer(x, y, mask=flag)
    assert torch.equal(e1, e2)
    assert rel_err(a.cpu(), e1.cpu()) < 0.5 and rel_err(a.cpu(), e1.cpu()) > 1e-3
    # same key: same masks, forward and backward
    import sparseattention_b200.fused_layer as fl
    layer.train()
    cfg = {"heads": H, "window": 16, "causal": True, "p": 0.1, "eps": 1e-5}
    key = torch.tensor([99], dtype=torch.int64, device="cuda")
    prm = list(fl.fused_layer_parameters(layer))
    xg = x.clone().requires_grad_()
    out1, _ = fl.FusedDecoderLayerFunction.apply(xg, y, cfg, key, *prm)
    out1.sum().backward()
    grad_b2 = layer.feed_forward.fc2.bias.grad.clone()
    with torch.no_grad():
        prm2 = list(prm)
        prm2[-1] = prm[-1] + 1.0
        out2, _ = fl.FusedDecoderLayerFunction.apply(x, y, cfg, key, *prm2)
        out3, _ = fl.FusedDecoderLayerFunction.apply(x, y, cfg, key, *prm)
    assert torch.equal(out3, out1.detach())
    mask_colsum = (out2 - out1.detach()).sum(dim=(0, 1))
    assert rel_err(grad_b2.cpu(), mask_colsum.cpu()) < 5e-3      # 1/(1-p) is rounded to bfloat16 in the backward's operand
    assert abs(float(mask_colsum.mean()) / (B * N) - 1.0) < 0.02


# ------------------------------------------------------------------------------------- logits ops
def test_logits_ops_golden(hsa, golden):
    """Span-attention weights against the tensor the reference's forward saves; the first prototype's cross logits
    against its own kernel (both run by the Triton interpreter when the fixture was made)."""
    from sparseattention_b200.ops import functional as F
    g = golden("logits_ops.npz")
    for tag in ("w_a", "w_b", "w_r0"):
        B, N, H, D, R = (int(v) for v in g[f"{tag}.meta"])
        for c in (1, 0):
            w = F.span_attention_logits(dev(g[f"{tag}.Q"]), dev(g[f"{tag}.K"]), R, bool(c), weights=True)
            assert w.shape == (B, N, H, 2 * R + 1 + int(math.log2(N)))
            assert rel_err(w.cpu(), g[f"{tag}.weights_c{c}"]) < 1e-5, (tag, c)
    B, N, H, D = (int(v) for v in g["v1.meta"])
    rs, rc = hsa.build_hierarchical_logits(dev(g["v1.ALL_Q"]), dev(g["v1.ALL_K"]), H, D, N)
    assert rel_err(rc.cpu(), g["v1.RES_CROSS"]) < 1e-5
    want_self, _ = orc.sibling_logits(torch.from_numpy(g["v1.ALL_Q"]), torch.from_numpy(g["v1.ALL_K"]), H, D, N)
    assert rel_err(rs.cpu(), want_self) < 1e-5


@pytest.mark.parametrize("case", [(1, 1, 1, 8, 2), (2, 16, 3, 24, 2), (1, 64, 2, 32, 5), (1, 64, 4, 64, 100),
                                  (2, 256, 3, 64, 8), (1, 512, 12, 64, 16), (1, 32, 1, 200, 3)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_span_logits_vs_oracle(hsa, case, causal, dtype):
    from sparseattention_b200.ops import functional as F
    B, N, H, D, R = case
    gen = torch.Generator().manual_seed(N + R)
    Q = torch.randn(B, N, H, D, generator=gen).to(dtype)
    K = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    want = orc.span_logits(Q, K, R, causal)
    got = F.span_attention_logits(Q.cuda(), K.cuda(), R, causal).cpu()
    inf = want == float("-inf")
    assert torch.equal(got == float("-inf"), inf)                                  # the same slots are masked
    assert rel_err(got.masked_fill(inf, 0), want.masked_fill(inf, 0)) < 1e-5      # float32 accumulation either way
    w = F.span_attention_logits(Q.cuda(), K.cuda(), R, causal, weights=True).cpu()
    assert rel_err(w, orc.span_logits(Q, K, R, causal, weights=True)) < 1e-5
    # the weights are those of the attention output: sum_c w_c v_c equals the forward
    V = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    rows, _ = orc.span_candidates(N, R, causal)
    out = torch.einsum("bnhc,bnchd->bnhd", w, V.float()[:, rows])
    fwd, _ = F.span_attention_forward(Q.cuda(), K.cuda(), V.cuda(), R, causal, algo=1)
    assert rel_err(fwd.float().cpu(), out) < TOL[dtype]


@pytest.mark.parametrize("shape", [(1, 3, 1, 8), (2, 31, 3, 16), (1, 127, 8, 64), (2, 15, 12, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sibling_logits_vs_oracle(hsa, shape, dtype):
    B, total, H, D = shape
    N = (total + 1) // 2
    gen = torch.Generator().manual_seed(total)
    Q = torch.randn(B, total, H * D, generator=gen).to(dtype)
    K = torch.randn(B, total, H * D, generator=gen).to(dtype)
    want_self, want_cross = orc.sibling_logits(Q, K, H, D, N)
    rs, rc = hsa.build_hierarchical_logits(Q.cuda(), K.cuda(), H, D, N)
    assert rs.dtype == torch.float32 and rs.shape == (B, N, H) and rc.shape == (B, total - 1, H)
    assert rel_err(rs.cpu(), want_self) < 1e-5 and rel_err(rc.cpu(), want_cross) < 1e-5


# ------------------------------------------------------------------------------------- the layer
def _module_pair(hsa, g, tag):
    B, N, H, Dh, R, seed, sub = (int(v) for v in g[f"{tag}.meta"])
    m = hsa.HierarchicalAttention(H * Dh, H, dropout=0.0, window_size=R).eval()
    m.load_state_dict({k: torch.from_numpy(g[f"{tag}.{k}"]) for k in WEIGHT_NAMES})
    return m.cuda(), (B, N, H, Dh, R)


@pytest.mark.parametrize("tag", ["tiny", "small", "wide_window"])
def test_layer_against_eager_reference_golden(hsa, golden, tag):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    g = golden("layer_eager.npz")
    m, (B, N, H, Dh, R) = _module_pair(hsa, g, tag)
    x = dev(g[f"{tag}.x"])
    xa = x.clone().requires_grad_()
    ya = hsa.generate_span_input_Y(x).detach().requires_grad_()
    y1 = m.cross_update_Y(xa, ya)
    y1.backward(dev(g[f"{tag}.gy"]))
    assert rel_err(y1.detach().cpu(), g[f"{tag}.y_new"]) < 1e-5
    assert rel_err(xa.grad.cpu(), g[f"{tag}.cuy_grad_x"]) < 1e-5
    assert rel_err(ya.grad.cpu(), g[f"{tag}.cuy_grad_y"]) < 1e-5
    for c in (1, 0):
        xb = x.clone().requires_grad_()
        yb = dev(g[f"{tag}.y_new"]).requires_grad_()
        o = m(xb, xb, xb, y=yb, mask=torch.ones(B, N, device="cuda") if c else None)
        o.backward(dev(g[f"{tag}.go"]))
        assert rel_err(o.detach().cpu(), g[f"{tag}.out_c{c}"]) < 1e-5
        assert rel_err(xb.grad.cpu(), g[f"{tag}.fwd_grad_x_c{c}"]) < 1e-5
        assert rel_err(yb.grad.cpu(), g[f"{tag}.fwd_grad_y_c{c}"]) < 1e-5


def test_layer_b2_h4_n512_fp32(hsa, golden):
    """fp32 layer, B2 H4 N512 Dh64, causal window 16: output and parent-node tensors, against the oracle on the
    full tensors and against the rows the reference's own eager layer produced (stored in the fixture)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    g = golden("layer_config1.npz")
    om, x, gy, go = config1_inputs(g)
    m = hsa.HierarchicalAttention(256, 4, dropout=0.0, window_size=16).eval()
    m.load_state_dict(om.state_dict())
    m = m.cuda()
    xc = x.cuda().requires_grad_()
    y0 = hsa.generate_span_input_Y(x.cuda()).detach().requires_grad_()
    y1 = m.cross_update_Y(xc, y0)
    y1.backward(gy.cuda())
    # against the oracle (full tensors)
    xo = x.clone().requires_grad_()
    yo0 = orc.generate_span_input_Y(x).requires_grad_()
    yo1 = om.cross_update_Y(xo, yo0)
    yo1.backward(gy)
    assert rel_err(y1.detach().cpu(), yo1.detach()) < 1e-5
    assert rel_err(xc.grad.cpu(), xo.grad) < 1e-5
    assert rel_err(y0.grad.cpu(), yo0.grad) < 1e-5
    mask = torch.ones(2, 512, device="cuda")
    xb = x.cuda().requires_grad_()
    yb = y1.detach().clone().requires_grad_()
    out = m(xb, xb, xb, y=yb, mask=mask)
    out.backward(go.cuda())
    xob = x.clone().requires_grad_()
    yob = yo1.detach().clone().requires_grad_()
    oo = om(xob, xob, xob, y=yob, mask=torch.ones(2, 512))
    oo.backward(go)
    assert rel_err(out.detach().cpu(), oo.detach()) < 1e-5
    assert rel_err(xb.grad.cpu(), xob.grad) < 1e-5
    assert rel_err(yb.grad.cpu(), yob.grad) < 1e-5
    # against the reference's own outputs (every `sub`-th row is stored)
    sub = int(g["config1.meta"][6])
    assert rel_err(y1.detach().cpu()[:, ::sub], g["config1.y_new"]) < 1e-5
    assert rel_err(xc.grad.cpu()[:, ::sub], g["config1.cuy_grad_x"]) < 1e-5
    assert rel_err(y0.grad.cpu()[:, ::sub], g["config1.cuy_grad_y"]) < 1e-5
    assert rel_err(out.detach().cpu()[:, ::sub], g["config1.out_c1"]) < 1e-5
    assert rel_err(xb.grad.cpu()[:, ::sub], g["config1.fwd_grad_x_c1"]) < 1e-5
    assert rel_err(yb.grad.cpu()[:, ::sub], g["config1.fwd_grad_y_c1"]) < 1e-5


def test_layer_b16_h8_n512_bf16(hsa):
    """The module at B16 H8 N512 Dh64, causal window 8, forward and backward, bf16 weights and activations,
    compared with the oracle layer run in float32 on the same bf16-rounded weights and inputs."""
    B, N, H, Dh, R = 16, 512, 8, 64, 8
    torch.manual_seed(2)
    om = orc.HierarchicalAttentionOracle(H * Dh, H, dropout=0.0, window_size=R).eval()
    for p in om.parameters():
        p.data = p.data.bfloat16().float()
    m = hsa.HierarchicalAttention(H * Dh, H, dropout=0.0, window_size=R).eval()
    m.load_state_dict(om.state_dict())
    m = m.cuda().bfloat16()
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(B, N, H * Dh, generator=gen).bfloat16()
    go = torch.randn(B, N, H * Dh, generator=gen).bfloat16()
    gy = torch.randn(B, N - 1, H * Dh, generator=gen).bfloat16()
    xo = x.float().requires_grad_()
    yo0 = orc.generate_span_input_Y(x.float()).requires_grad_()
    yo1 = om.cross_update_Y(xo, yo0)
    yo1.backward(gy.float())
    xc = x.cuda().requires_grad_()
    yc0 = hsa.generate_span_input_Y(x.cuda()).detach().requires_grad_()
    yc1 = m.cross_update_Y(xc, yc0)
    yc1.backward(gy.cuda())
    assert rel_err(yc1.detach().float().cpu(), yo1.detach()) < 2e-2
    assert rel_err(xc.grad.float().cpu(), xo.grad) < 2e-2
    assert rel_err(yc0.grad.float().cpu(), yo0.grad) < 2e-2
    y_in = yo1.detach().bfloat16()
    xob = x.float().requires_grad_()
    yob = y_in.float().requires_grad_()
    oo = om(xob, xob, xob, y=yob, mask=torch.ones(B, N))
    oo.backward(go.float())
    xcb = x.cuda().requires_grad_()
    ycb = y_in.cuda().requires_grad_()
    oc = m(xcb, xcb, xcb, y=ycb, mask=torch.ones(B, N, device="cuda"))
    oc.backward(go.cuda())
    assert rel_err(oc.detach().float().cpu(), oo.detach()) < 2e-2
    assert rel_err(xcb.grad.float().cpu(), xob.grad) < 2e-2
    assert rel_err(ycb.grad.float().cpu(), yob.grad) < 2e-2


def test_module_api_surface(hsa):
    m = hsa.HierarchicalAttention(64, 4, dropout=0.1, window_size=3).cuda()
    assert sorted(n for n, _ in m.named_parameters()) == sorted(WEIGHT_NAMES)
    x = torch.randn(2, 16, 64, device="cuda")
    y = hsa.generate_span_input_Y(x)
    out, attn = m(x, x, x, y=m.cross_update_Y(x, y), mask=torch.ones(2, 16, device="cuda"), return_attention=True)
    assert out.shape == (2, 16, 64) and attn is None
    assert m.cached_seq_len == 16 and m.cached_is_causal is True and m.sizes == [8, 4, 2, 1]
    # dense branch when no parents are given
    dense = m.eval()(x, x, x)
    assert dense.shape == (2, 16, 64)
    # a second sequence length through the same module
    x2 = torch.randn(1, 64, 64, device="cuda")
    y2 = m.cross_update_Y(x2, hsa.generate_span_input_Y(x2))
    assert y2.shape == (1, 63, 64) and m(x2, x2, x2, y=y2, mask=None).shape == (1, 64, 64)


def test_language_model_against_oracle_layers(hsa):
    """The LM that calls the layer (6 -> 2 layers, small widths), fp32: logits, loss and a few gradients
    against the same model built around the CPU oracle layer."""
    from sparseattention_b200.lm import TransformerLM, lm_loss, zipf_tokens
    torch.backends.cuda.matmul.allow_tf32 = False
    vocab, d, heads, ff, layers, N = 211, 64, 4, 128, 2, 64      # 211 pads to 256 rows
    torch.manual_seed(5)
    ref = TransformerLM(vocab, d, heads, ff, layers, dropout=0.0, window_size=4,
                        attention_cls=orc.HierarchicalAttentionOracle, span_init=orc.generate_span_input_Y).eval()
    torch.manual_seed(5)
    ours = TransformerLM(vocab, d, heads, ff, layers, dropout=0.0, window_size=4).eval()
    ours.load_state_dict(ref.state_dict())
    ours = ours.cuda()
    tokens = zipf_tokens(2, N + 1, vocab, seed=9)
    lr = orc.lm_loss_reference(ref, tokens)
    lr.backward()
    lo = lm_loss(ours, tokens.cuda())
    lo.backward()
    assert abs(float(lo) - float(lr)) < 1e-5 * abs(float(lr))
    assert rel_err(ours(tokens[:, :-1].cuda()).detach().cpu(), ref(tokens[:, :-1]).detach()) < 1e-5
    for name in ("embedding.weight", "layers.0.self_attn.Wk_y.weight", "layers.1.self_attn.Wq_x.weight",
                 "layers.0.norm_y.weight", "layers.1.feed_forward.fc1.weight"):
        g_ours = dict(ours.named_parameters())[name].grad.cpu()
        g_ref = dict(ref.named_parameters())[name].grad
        assert rel_err(g_ours, g_ref) < 2e-5, name


def test_language_model_bf16_autocast_training_step(hsa):
    """One bf16-autocast training step of the LM at the benchmarked widths (d_model 512, 8 heads, FFN 2048,
    window 16, vocabulary 50257; 2 layers, one sequence of 2048 tokens, no dropout): loss and a few gradients
    against the same model around the CPU oracle layer, run in float32 on bf16-rounded Linear weights.
    Tolerance 2e-2 (loss: relative)."""
    from sparseattention_b200.lm import TransformerLM, lm_loss, zipf_tokens
    vocab, d, heads, ff, layers, N = 50257, 512, 8, 2048, 2, 2048
    torch.manual_seed(11)
    ours = TransformerLM(vocab, d, heads, ff, layers, dropout=0.0, window_size=16).train()
    ref = TransformerLM(vocab, d, heads, ff, layers, dropout=0.0, window_size=16,
                        attention_cls=orc.HierarchicalAttentionOracle, span_init=orc.generate_span_input_Y).train()
    ref.load_state_dict(ours.state_dict())
    with torch.no_grad():
        for mod in ref.modules():
            if isinstance(mod, torch.nn.Linear):               # autocast rounds these operands to bf16
                mod.weight.copy_(mod.weight.bfloat16().float())
    ours = ours.cuda()
    tokens = zipf_tokens(1, N + 1, vocab, seed=13)
    lr = orc.lm_loss_reference(ref, tokens)
    lr.backward()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        lo = lm_loss(ours, tokens.cuda())
    lo.backward()
    assert abs(float(lo) - float(lr)) < 2e-2 * abs(float(lr)), (float(lo), float(lr))
    got, want = dict(ours.named_parameters()), dict(ref.named_parameters())
    for name in ("embedding.weight", "layers.0.self_attn.Wk_y.weight", "layers.1.self_attn.Wq_x.weight",
                 "layers.0.norm_y.weight", "layers.1.feed_forward.fc2.weight"):
        assert rel_err(got[name].grad.float().cpu(), want[name].grad) < 2e-2, name


def test_language_model_weight_copies_follow_the_weights(hsa):
    """The model keeps bfloat16 copies of its layers' weights for the fused layers and refreshes them at every forward: after
    a weight changes in place (an optimizer step) the fused path has to see the new value, like the module-by-module path."""
    from sparseattention_b200.lm import TransformerLM
    torch.manual_seed(5)
    model = TransformerLM(1000, 256, 4, 512, 2, dropout=0.0, window_size=8).cuda().eval()
    tokens = torch.randint(0, 1000, (2, 256), device="cuda")

    def run(fused):
        for layer in model.layers:
            layer.fused = fused
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return model(tokens, hidden_only=True).float()

    before = run(True)
    assert getattr(model, "_w16_cache", None) is not None           # the fused path ran and built its copies
    with torch.no_grad():
        model.layers[0].feed_forward.fc1.weight.mul_(1.5)
        model.layers[1].self_attn.Wv_x.weight.add_(0.05)
    after_fused, after_eager = run(True), run(False)
    assert rel_err(after_fused.cpu(), after_eager.cpu()) < 2e-2
    assert rel_err(after_fused.cpu(), before.cpu()) > 5e-2          # the change is large enough to tell stale copies apart


# ------------------------------------------------------------------------------------- incremental decoding
@pytest.mark.parametrize("case", [(2, 16, 3, 24, 2), (1, 64, 2, 32, 5), (3, 256, 4, 64, 16), (1, 1024, 12, 64, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_span_attention_decode_vs_oracle(hsa, case, dtype):
    """The single-leaf op against the oracle's causal span attention evaluated at that leaf; rows of later leaves
    and of nodes that are not complete yet hold NaN in the cache, so reading any of them would show."""
    from sparseattention_b200.ops import functional as F
    B, N, H, D, R = case
    gen = torch.Generator().manual_seed(N * 3 + R)
    Q = torch.randn(B, N, H, D, generator=gen).to(dtype)
    K = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    V = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype)
    for n in sorted({0, 1, 2, 5, N // 2 - 1, N // 2, N - 2, N - 1}):
        if n < 0 or n >= N:
            continue
        want = orc.hierarchical_attention(Q, K, V, R, True, leaves=torch.tensor([n]))[:, 0]
        Kc, Vc = K.clone(), V.clone()
        Kc[:, n + 1:N] = float("nan")
        Vc[:, n + 1:N] = float("nan")
        for lvl in range(1, int(math.log2(N)) + 1):     # a node is complete when the last leaf under it is <= n
            base = 2 * N - (N >> (lvl - 1))
            for j in range(N >> lvl):
                if (j + 1) * (1 << lvl) - 1 > n:
                    Kc[:, base + j] = float("nan")
                    Vc[:, base + j] = float("nan")
        got = F.span_attention_decode(Q[:, n].cuda(), Kc.cuda(), Vc.cuda(), n, R)
        assert rel_err(got.float().cpu(), want) < TOL[dtype], n


def test_incremental_decoder_matches_full_forward(hsa):
    """IncrementalDecoder logits at every position equal the full forward's (fp32), for a cache exactly as long as the
    sequence and for a longer one; generate() returns prompt + sampled tokens."""
    from sparseattention_b200.lm import IncrementalDecoder, TransformerLM, generate, zipf_tokens
    torch.backends.cuda.matmul.allow_tf32 = False
    vocab, d, heads, ff, layers, N = 211, 64, 4, 128, 2, 32
    torch.manual_seed(7)
    model = TransformerLM(vocab, d, heads, ff, layers, dropout=0.1, window_size=4).cuda().eval()
    tokens = zipf_tokens(2, N, vocab, seed=3).cuda()
    with torch.no_grad():
        full = model(tokens)
    for capacity in (N, 2 * N):
        dec = IncrementalDecoder(model, 2, capacity)
        for n in range(N):
            logits = dec.step(tokens[:, n])
            assert rel_err(logits.cpu(), full[:, n].cpu()) < 1e-4, (capacity, n)
    # a prefix of a longer sequence sees the same logits (causality of the whole model)
    with torch.no_grad():
        half = model(tokens[:, : N // 2])
    assert rel_err(half.cpu(), full[:, : N // 2].cpu()) < 1e-4
    out = generate(model, tokens[0, :5], max_len=6, eos_token=None, generator=torch.Generator(device="cuda").manual_seed(1))
    assert out.shape == (1, 11) and torch.equal(out[0, :5], tokens[0, :5]) and int(out.max()) < vocab


# ------------------------------------------------------------------------------------- dropout
def _probe_module(hsa, d, H, p, R):
    """A layer whose projections are zero (queries, keys: uniform attention weights) or the identity
    (values, output projections), so its outputs show the dropout masks directly."""
    m = hsa.HierarchicalAttention(d, H, dropout=p, window_size=R).cuda()
    with torch.no_grad():
        for name in ("Wq_y", "Wk_y", "Wq_x", "Wk_x"):
            getattr(m, name).weight.zero_()
        for name in ("Wv_y", "Wv_x", "out_proj_y", "out_proj_x"):
            getattr(m, name).weight.copy_(torch.eye(d))
        m.out_proj_y.bias.zero_()
        m.out_proj_x.bias.zero_()
    return m


def test_dropout_on_child_values_bottom_up(hsa):
    """cross_update_Y in training mode, p = 0.1: the children's values are dropped (leaf values twice, as
    hierarchical_attention/modules/attention.py:117,135 of the reference does; values of higher levels once),
    kept entries are scaled by 1/(1-p) per application, and the mean is preserved."""
    torch.backends.cuda.matmul.allow_tf32 = False
    p, B, N, d, H = 0.1, 4, 1024, 64, 4
    m = _probe_module(hsa, d, H, p, 2).train()
    x = torch.ones(B, N, d, device="cuda")
    y = m.cross_update_Y(x, torch.zeros(B, N - 1, d, device="cuda"))
    keep = 1.0 - p
    # level 1: (1/3) (0 + a + b), a and b in {0, 1/keep^2}
    lvl0 = y[:, : N // 2].double() * 3 * keep * keep
    k0 = lvl0.round()
    assert float((lvl0 - k0).abs().max()) < 1e-4 and set(k0.unique().tolist()) <= {0.0, 1.0, 2.0}
    both, none = float((k0 == 2).double().mean()), float((k0 == 0).double().mean())
    assert abs(both - keep ** 4) < 0.01 and abs(none - (1 - keep * keep) ** 2) < 0.005
    # level 2: (1/3) (0 + a' + b'), a', b' = level-1 outputs dropped once
    lvl1 = y[:, N // 2: N // 2 + N // 4].double() * 3 * keep * 3 * keep * keep
    k1 = lvl1.round()
    assert float((lvl1 - k1).abs().max()) < 1e-3 and float(k1.max()) <= 4.0
    assert abs(float(y[:, : N // 2].mean()) - 2 / 3) < 0.01
    assert abs(float(y[:, N // 2: N // 2 + N // 4].mean()) - 4 / 9) < 0.01
    zero1 = (p + keep * (1 - keep * keep) ** 2) ** 2
    assert abs(float((k1 == 0).double().mean()) - zero1) < 0.005
    # evaluation mode: no dropout at all
    ye = m.eval().cross_update_Y(x, torch.zeros(B, N - 1, d, device="cuda"))
    assert float((ye[:, : N // 2] - 2 / 3).abs().max()) < 1e-5


def test_dropout_leaves_queries_and_keys_alone_bottom_up(hsa):
    """With child values that are exactly zero (x in the null space of Wv_y) the first level of cross_update_Y is
    a function of the queries, the keys and the parents' own values only: training mode must reproduce the
    evaluation-mode result bit for bit, i.e. no mask touches Q, K or the parents' values."""
    torch.backends.cuda.matmul.allow_tf32 = False
    B, N, d, H = 2, 256, 64, 4
    gen = torch.Generator().manual_seed(21)
    m = hsa.HierarchicalAttention(d, H, dropout=0.1, window_size=2).cuda()
    with torch.no_grad():
        m.Wk_y.weight.copy_(torch.eye(d))
        half = torch.zeros(d)
        half[: d // 2] = 1.0
        m.Wv_y.weight.copy_(torch.diag(half))
        m.out_proj_y.weight.copy_(torch.eye(d))
        m.out_proj_y.bias.zero_()
    x = torch.randn(B, N, d, generator=gen)
    x[..., : d // 2] = 0.0
    y_in = torch.randn(B, N - 1, d, generator=gen)
    yt = m.train().cross_update_Y(x.cuda(), y_in.cuda())
    ye = m.eval().cross_update_Y(x.cuda(), y_in.cuda())
    assert float(ye[:, : N // 2].abs().max()) > 0.1
    assert torch.equal(yt[:, : N // 2], ye[:, : N // 2])
    assert not torch.equal(yt[:, N // 2:], ye[:, N // 2:])          # higher levels do see dropped values


def test_dropout_on_values_top_down(hsa):
    """update_X_from_Y in training mode, p = 0.1: values of leaves and parents are dropped once (kept entries
    scaled by 1/(1-p)), attention weights are not; the mean is preserved."""
    torch.backends.cuda.matmul.allow_tf32 = False
    p, B, N, d, H, R = 0.1, 4, 1024, 64, 4, 5
    m = _probe_module(hsa, d, H, p, R).train()
    x = torch.ones(B, N, d, device="cuda")
    y = torch.ones(B, N - 1, d, device="cuda")
    out = m.update_X_from_Y(x, y, mask=torch.ones(1, device="cuda"))
    n = torch.arange(N)
    count = (torch.minimum(n, torch.tensor(R)) + 1 + torch.tensor([bin(int(i)).count("1") for i in n])).double()
    k = out.double().cpu() * count[None, :, None] * (1 - p)
    assert float((k - k.round()).abs().max()) < 1e-3
    assert float((k.round() - count[None, :, None]).max()) <= 0 and float(k.min()) > -1e-3
    assert abs(float(out.mean()) - 1.0) < 0.01
    assert abs(float((k.round() / count[None, :, None]).mean()) - (1 - p)) < 0.01
    # the weights see no mask: the mean over many identical sequences approaches the evaluation-mode output
    gen = torch.Generator().manual_seed(22)
    Bm, Nm, dm = 4096, 32, 32
    mm = hsa.HierarchicalAttention(dm, 2, dropout=p, window_size=3).cuda()
    xs = torch.randn(1, Nm, dm, generator=gen).cuda().expand(Bm, Nm, dm).contiguous()
    ys = torch.randn(1, Nm - 1, dm, generator=gen).cuda().expand(Bm, Nm - 1, dm).contiguous()
    flag = torch.ones(1, device="cuda")
    with torch.no_grad():
        mean_train = mm.train().update_X_from_Y(xs, ys, mask=flag).mean(dim=0)
        want = mm.eval().update_X_from_Y(xs[:1], ys[:1], mask=flag)[0]
    from tests.conftest import max_rel_err
    assert max_rel_err(mean_train.cpu(), want.cpu()) < 0.03


@pytest.mark.parametrize("M,V,Vp", [(7, 5, 5), (33, 211, 256), (16, 50257, 50304), (4, 1000, 1001)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("eps", [0.0, 0.1])
def test_cross_entropy_vs_torch(hsa, M, V, Vp, dtype, eps):
    from sparseattention_b200.ops.loss import cross_entropy
    gen = torch.Generator().manual_seed(M + V)
    logits = (torch.randn(M, Vp, generator=gen) * 3).to(dtype)
    targets = torch.randint(0, V, (M,), generator=gen)
    targets[0] = -100                                   # an ignored row
    ref_in = logits[:, :V].double().clone().requires_grad_()          # float64 on the same rounded logits
    ref = torch.nn.functional.cross_entropy(ref_in, targets, label_smoothing=eps, ignore_index=-100)
    ref.backward()
    x = logits.cuda().requires_grad_()
    out = cross_entropy(x, targets.cuda(), V, label_smoothing=eps, ignore_index=-100)
    out.backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert abs(float(out.detach()) - float(ref.detach())) <= 1e-5 * abs(float(ref.detach())) + 1e-6
    assert rel_err(x.grad[:, :V].float().cpu(), ref_in.grad) < tol
    assert float(x.grad[:, V:].abs().sum()) == 0.0 and float(x.grad[0].abs().sum()) == 0.0


@pytest.mark.parametrize("M,d,V,Vp", [(300, 64, 211, 256), (1000, 512, 50257, 50304), (129, 128, 1000, 1000)])
@pytest.mark.parametrize("eps", [0.0, 0.1])
def test_linear_cross_entropy_vs_torch(hsa, M, d, V, Vp, eps):
    """LM head + loss in one pass against float64 F.linear + F.cross_entropy on the same bf16-rounded operands:
    loss, and the gradients of x, weight and bias; the loss-only path (no logits written) gives the same value."""
    from sparseattention_b200.ops.loss import linear_cross_entropy
    gen = torch.Generator().manual_seed(M + V)
    x = torch.randn(M, d, generator=gen).bfloat16()
    w = (torch.randn(Vp, d, generator=gen) * 0.05).bfloat16()
    b = torch.randn(Vp, generator=gen) * 0.1
    targets = torch.randint(0, V, (M,), generator=gen)
    targets[3] = -100
    xr, wr, br = x.double().requires_grad_(), w.double().requires_grad_(), b.double().requires_grad_()
    ref = torch.nn.functional.cross_entropy(torch.nn.functional.linear(xr, wr, br)[:, :V], targets, label_smoothing=eps, ignore_index=-100)
    ref.backward()
    xc, wc, bc = x.cuda().requires_grad_(), w.cuda().requires_grad_(), b.cuda().requires_grad_()
    out = linear_cross_entropy(xc, wc, bc, targets.cuda(), V, label_smoothing=eps, ignore_index=-100)
    out.backward()
    assert abs(float(out.detach()) - float(ref.detach())) < 2e-3 * abs(float(ref.detach()))     # logits rounded to bf16
    assert rel_err(xc.grad.float().cpu(), xr.grad) < 2e-2
    assert rel_err(wc.grad.float().cpu()[:V], wr.grad[:V]) < 2e-2 and float(wc.grad[V:].abs().max() if Vp > V else 0) == 0.0
    assert rel_err(bc.grad.cpu()[:V], br.grad[:V]) < 2e-2
    with torch.no_grad():
        loss_only = linear_cross_entropy(x.cuda(), w.cuda(), b.cuda(), targets.cuda(), V, label_smoothing=eps, ignore_index=-100)
    assert abs(float(loss_only) - float(out.detach())) < 1e-6 * abs(float(out.detach()))
    bad = targets.clone()
    bad[5] = V + 3
    with torch.no_grad():
        assert bool(linear_cross_entropy(x.cuda(), w.cuda(), b.cuda(), bad.cuda(), V).isnan())


def test_host_entry_point_matches_device_path(hsa):
    """hierarchical_attention_from_host (chunked, stream-overlapped) gives the device path's bits."""
    from sparseattention_b200.ops import functional as F
    gen = torch.Generator().manual_seed(4)
    B, N, H, D, R = 5, 256, 4, 64, 8
    Q = torch.randn(B, N, H, D, generator=gen).bfloat16().pin_memory()
    K = torch.randn(B, 2 * N - 1, H, D, generator=gen).bfloat16().pin_memory()
    V = torch.randn(B, 2 * N - 1, H, D, generator=gen).bfloat16().pin_memory()
    want, _ = F.span_attention_forward(Q.cuda(), K.cuda(), V.cuda(), R, True, need_lse=False)
    for chunks in (1, 2, 8):
        got = F.hierarchical_attention_from_host(Q, K, V, R, True, chunks=chunks)
        torch.cuda.synchronize()
        assert torch.equal(got, want.cpu())


@pytest.mark.parametrize("shape", [(3, 128), (4, 37, 256), (2, 100, 384), (8, 513, 512), (2, 16, 768)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_vs_torch(hsa, shape, dtype):
    from sparseattention_b200.ops.norm import LayerNorm
    gen = torch.Generator().manual_seed(shape[-1])
    d = shape[-1]
    x = (torch.randn(*shape, generator=gen) * 2 + 0.5).to(dtype)
    dy = torch.randn(*shape, generator=gen).to(dtype)
    ref = torch.nn.LayerNorm(d).double()
    with torch.no_grad():
        ref.weight.copy_(torch.randn(d, generator=gen))
        ref.bias.copy_(torch.randn(d, generator=gen))
    ours = LayerNorm(d)
    ours.load_state_dict({k: v.float() for k, v in ref.state_dict().items()})
    ours = ours.cuda()
    xr = x.double().requires_grad_()
    ref(xr).backward(dy.double())
    xo = x.cuda().requires_grad_()
    yo = ours(xo)
    yo.backward(dy.cuda())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert yo.dtype == dtype
    assert rel_err(yo.detach().float().cpu(), ref(x.double()).detach()) < tol
    assert rel_err(xo.grad.float().cpu(), xr.grad) < tol
    assert rel_err(ours.weight.grad.cpu(), ref.weight.grad) < (1e-5 if dtype == torch.float32 else 2e-2)
    assert rel_err(ours.bias.grad.cpu(), ref.bias.grad) < (1e-5 if dtype == torch.float32 else 2e-2)
    # widths the kernel does not take still work (library fallback)
    odd = LayerNorm(100).cuda()
    assert odd(torch.randn(3, 100, device="cuda")).shape == (3, 100)


def test_forward_bulk_copy_waits_never_expire(hsa):
    """The TMA-staged kernels bound their mbarrier waits; in normal operation no CTA hits the bound."""
    from sparseattention_b200 import _lib
    from sparseattention_b200.ops import functional as F
    before = _lib.wait_expired_count()
    q = torch.randn(2, 4096, 4, 128, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(2, 8191, 4, 128, device="cuda", dtype=torch.bfloat16)
    out, lse = F.span_attention_forward(q, kv, kv, 16, True, algo=4)
    F.span_attention_backward(q, kv, kv, out, lse, torch.randn_like(out), 16, True)
    assert _lib.wait_expired_count() == before


def test_bounded_wait_gives_up_visibly(hsa, monkeypatch):
    """The give-up path of the TMA-staged kernels, made to run without anything hanging or faulting: the test
    hook shortens the wait to about a millisecond and makes each CTA's first barrier expect 64 bytes more than
    its copies deliver, so all copies complete, the barrier does not, and the (single) CTA of each launch gives
    up.  It must return, count itself, and leave NaN instead of results; the Python binding's debug mode turns
    that into an exception."""
    from sparseattention_b200 import _lib
    from sparseattention_b200.ops import functional as F
    lib = _lib.load()
    gen = torch.Generator().manual_seed(31)

    def inputs(N):
        q = torch.randn(1, N, 1, 128, generator=gen).bfloat16().cuda()
        k = torch.randn(1, 2 * N - 1, 1, 128, generator=gen).bfloat16().cuda()
        v = torch.randn(1, 2 * N - 1, 1, 128, generator=gen).bfloat16().cuda()
        return q, k, v

    q128, k128, v128 = inputs(128)
    q64, k64, v64 = inputs(64)
    good_out, good_lse = F.span_attention_forward(q64, k64, v64, 16, True, algo=3)
    go = torch.randn_like(good_out)
    good = F.span_attention_backward(q64, k64, v64, good_out, good_lse, go, 16, True, algo=4)
    before = _lib.wait_expired_count()
    try:
        _lib.check(lib.hsa_debug_wait_test(2_000_000, 64), "hsa_debug_wait_test")
        out, lse = F.span_attention_forward(q128, k128, v128, 16, True, algo=4)          # 128-leaf forward, one CTA
        assert bool(out.isnan().all()) and bool(lse.isnan().all())
        assert _lib.wait_expired_count() == before + 1
        out, lse = F.span_attention_forward(q64, k64, v64, 16, True, algo=3)             # 64-leaf forward, one CTA
        assert bool(out.isnan().all()) and bool(lse.isnan().all())
        assert _lib.wait_expired_count() == before + 2
        dq, dk, dv = F.span_attention_backward(q64, k64, v64, good_out, good_lse, go, 16, True, algo=4)   # 8-warp backward
        assert bool(dq.isnan().all())
        assert _lib.wait_expired_count() == before + 3
        monkeypatch.setattr(_lib, "DEBUG", True)
        _lib._expired_seen[torch.cuda.current_device()] = _lib.wait_expired_count()
        with pytest.raises(_lib.HsaError, match="gave up waiting"):
            F.span_attention_forward(q128, k128, v128, 16, True, algo=4)
    finally:
        _lib.check(lib.hsa_debug_wait_test(2_000_000_000, 0), "hsa_debug_wait_test")
    monkeypatch.setattr(_lib, "DEBUG", False)
    # back to normal: same bits as before the hook was set
    out, lse = F.span_attention_forward(q64, k64, v64, 16, True, algo=3)
    assert torch.equal(out, good_out) and torch.equal(lse, good_lse)
    again = F.span_attention_backward(q64, k64, v64, good_out, good_lse, go, 16, True, algo=4)
    assert all(torch.equal(a, b) for a, b in zip(again, good))


def test_cross_entropy_flags_corrupt_targets(hsa):
    """A target outside [0, V) that is not the ignore index yields a NaN loss instead of a plausible number."""
    from sparseattention_b200.ops.loss import cross_entropy
    logits = torch.randn(4, 16, device="cuda")
    targets = torch.tensor([1, 2, 99, 3], device="cuda")
    assert bool(cross_entropy(logits, targets, 10).isnan())
    targets[2] = -100
    assert bool(cross_entropy(logits, targets, 10).isfinite())


def test_backward_without_workspace_when_none_is_needed(hsa):
    """hsa_span_attn_bwd accepts a null workspace when the size query returns 0 (N = 64 tensor-core case) and reports
    the real argument error (dtype), not a workspace error, for float32 with a tensor-core algo."""
    from sparseattention_b200 import _lib
    from sparseattention_b200.ops import functional as F
    lib = _lib.load()
    q = torch.randn(1, 64, 2, 64, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(1, 127, 2, 64, device="cuda", dtype=torch.bfloat16)
    out, lse = F.span_attention_forward(q, kv, kv, 8, True)
    go = torch.randn_like(out)
    assert int(lib.hsa_span_attn_bwd_workspace_bytes(1, 64, 2, 64, 8, 1, _lib.HSA_BF16, 2)) == 0
    dq, dk, dv = torch.empty_like(q), torch.empty_like(kv), torch.empty_like(kv)
    rc = lib.hsa_span_attn_bwd(*(_lib.rows_view(t) for t in (q, kv, kv, out)), lse.data_ptr(),
                               *(_lib.rows_view(t) for t in (go, dq, dk, dv)), None, 0,
                               1, 64, 2, 64, 8, 1, _lib.HSA_BF16, 2, _lib.stream_ptr(q.device))
    _lib.check(rc, "hsa_span_attn_bwd")
    want = F.span_attention_backward(q, kv, kv, out, lse, go, 8, True, algo=2)
    assert torch.equal(dq, want[0]) and torch.equal(dk, want[1]) and torch.equal(dv, want[2])
    qf, kvf = q.float(), kv.float()
    rc = lib.hsa_span_attn_bwd(*(_lib.rows_view(t) for t in (qf, kvf, kvf, out.float())), lse.data_ptr(),
                               *(_lib.rows_view(t) for t in (go.float(), qf.clone(), kvf.clone(), kvf.clone())), None, 0,
                               1, 64, 2, 64, 8, 1, _lib.HSA_F32, 2, _lib.stream_ptr(q.device))
    assert rc == -1 and b"workspace" not in lib.hsa_last_error()
