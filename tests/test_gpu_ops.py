"""GPU parity of the operators, through the C ABI (libelb.so), against the CPU oracle on the same seeded inputs.

Bars: decoded weights, limb splits and int32 limb sums bit-exact; fp32 matvec / matmul outputs within 1e-5 of the
oracle's el::matvec restatement, relative to the largest |y| of the call (written in REL_TOL below) and adjudicated by
a float64 dot product of the decoded row when the oracle's own fp32 rounding is the larger error.
"""
import numpy as np
import pytest

import oracle_lib as ol
from exactinfer_b200 import synth

pytestmark = pytest.mark.gpu
REL_TOL = 1e-5
QTYPES = (synth.Q4_K, synth.Q6_K, synth.Q8_0)


@pytest.fixture(scope="module")
def elb():
    import exactinfer_b200 as e
    ok, why = e.cuda_available()
    assert ok, f"CUDA path unavailable: {why}"
    return e


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def rel_err(y, ref):
    return float(np.abs(y.astype(np.float64) - ref.astype(np.float64)).max() / max(np.abs(ref).max(), 1e-30))


def check_matvec(y, w_bytes, t, rows, n, x):
    ref = ol.matvec(t, rows, n, w_bytes, x)
    e = rel_err(y, ref)
    if e > REL_TOL:  # adjudicate against exact arithmetic on the decoded weights
        deq = ol.dequant_rows(t, rows, n, w_bytes).astype(np.float64)
        exact = deq @ x.astype(np.float64)
        e_gpu = np.abs(y - exact).max() / np.abs(exact).max()
        e_ref = np.abs(ref - exact).max() / np.abs(exact).max()
        assert e_gpu <= max(REL_TOL, e_ref), (e, e_gpu, e_ref)
    return e


@pytest.mark.parametrize("t", QTYPES + (synth.F16,))
@pytest.mark.parametrize("rows,n", ((16, 256), (37, 512), (130, 1024)))
def test_decoded_rows_bit_exact(elb, t, rows, n):
    rng = np.random.default_rng(rows * 7 + t)
    wb = synth.rand_weight(rng, t, rows, n)
    w = elb.Weight(t, rows, n, wb)
    got = w.get_rows(0, rows)
    assert np.array_equal(bits(got), bits(ol.dequant_rows(t, rows, n, wb)))
    one = elb.get_row(w, rows - 1)
    assert np.array_equal(bits(one), bits(ol.dequant_rows(t, rows, n, wb, rows - 1, 1)[0]))
    with pytest.raises(IndexError):
        w.get_rows(rows, 1)


@pytest.mark.parametrize("nl", (3, 4))
def test_limb_split_bit_exact(elb, nl):
    rng = np.random.default_rng(nl)
    x = rng.normal(size=(5, 768)).astype(np.float32)
    x[1] *= 1e-12
    x[2] *= 3e9
    x[3] = 0.0
    limbs, inv = elb.split_limbs(x, nl)
    for b in range(5):
        want, winv, _ = ol.split_limbs(x[b], nl)
        assert np.array_equal(limbs[:, b, :], want), b
        assert inv[b] == np.float32(winv)


@pytest.mark.parametrize("t", QTYPES)
@pytest.mark.parametrize("rows,n", ((16, 256), (40, 768), (200, 2048)))
def test_limb_sums_bit_exact(elb, t, rows, n):
    rng = np.random.default_rng(rows + n + t)
    wb = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=n).astype(np.float32)
    w = elb.Weight(t, rows, n, wb)
    for nl in (3, 4):
        P, I, J = w.limb_sums(x, nl)
        limbs, _, _ = ol.split_limbs(x, nl)
        assert np.array_equal(P, ol.limb_partials(t, rows, n, wb, limbs)), "sub-block partials"
        wI, wJ = ol.limb_block_sums(t, rows, n, wb, limbs)
        assert np.array_equal(I, wI), "block sums"
        assert np.array_equal(J, wJ), "min-term sums"


@pytest.mark.parametrize("t", QTYPES + (synth.F16,))
@pytest.mark.parametrize("rows,n", ((16, 256), (37, 512), (300, 1024), (1000, 2560), (2560, 4096)))
def test_matvec_matches_oracle(elb, t, rows, n):
    rng = np.random.default_rng(rows ^ n ^ t)
    wb = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=n).astype(np.float32)
    w = elb.Weight(t, rows, n, wb)
    y = elb.matvec(w, x, 4)
    check_matvec(y, wb, t, rows, n, x)
    y2 = elb.matvec(w, x, 4)
    assert np.array_equal(bits(y), bits(y2)), "matvec must be deterministic"
    if t != synth.F16:
        check_matvec(elb.matvec(w, x, 3), wb, t, rows, n, x)


def test_matvec_edge_inputs(elb):
    rng = np.random.default_rng(3)
    rows, n = 48, 512
    wb = synth.rand_weight(rng, synth.Q4_K, rows, n)
    w = elb.Weight(synth.Q4_K, rows, n, wb)
    assert not elb.matvec(w, np.zeros(n, np.float32)).any()
    x = np.zeros(n, np.float32)
    x[17] = -3.5e-20
    check_matvec(elb.matvec(w, x), wb, synth.Q4_K, rows, n, x)
    x = (rng.normal(size=n) * 1e15).astype(np.float32)
    check_matvec(elb.matvec(w, x), wb, synth.Q4_K, rows, n, x)
    with pytest.raises(ValueError):
        elb.matvec(w, np.zeros(n + 1, np.float32))


@pytest.mark.parametrize("t", QTYPES + (synth.F16,))
@pytest.mark.parametrize("b", (2, 16, 24, 33, 64, 70))  # 16, 24, 64: the narrow token tiles of the tensor-core kernel
def test_matmul_matches_oracle(elb, t, b):
    rng = np.random.default_rng(b + t)
    rows, n = 200, 1024
    wb = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=(b, n)).astype(np.float32)
    x[0] *= 50.0
    w = elb.Weight(t, rows, n, wb, planes=True)
    y = w.matmul(x, 4)
    for i in range(b):
        check_matvec(y[i], wb, t, rows, n, x[i])
    if t != synth.F16 and b in (16, 24):
        y3 = w.matmul(x, 3)
        for i in range(0, b, 5):
            check_matvec(y3[i], wb, t, rows, n, x[i])


@pytest.mark.parametrize("t,nl,b", ((synth.Q4_K, 4, 560), (synth.Q6_K, 3, 530)))
def test_matmul_whole_waves_and_shared_tiles(elb, t, nl, b):
    """More output tiles than SMs: the tensor-core kernel computes whole waves of tiles, cuts the remaining tiles by
    256-blocks over all CTAs and adds the partial sums of a shared tile in a fixed order (twice the same bits)."""
    rng = np.random.default_rng(b)
    rows, n = 1700, 768  # 14 row tiles x 12 (48 tokens) or 9 (64 tokens) token tiles of 3 blocks each
    wb = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=(b, n)).astype(np.float32)
    x[5] *= 1e4
    w = elb.Weight(t, rows, n, wb, planes=True)
    y = w.matmul(x, nl)
    for i in [5] + list(range(0, b, 37)) + [b - 1]:
        check_matvec(y[i], wb, t, rows, n, x[i])
    assert np.array_equal(bits(y), bits(w.matmul(x, nl))), "matmul must be deterministic"


def test_rmsnorm_matches_oracle(elb):
    rng = np.random.default_rng(8)
    for n in (128, 2560):
        x = (rng.normal(size=(3, n)) * 4).astype(np.float32)
        w = synth.rand_norm(rng, n)
        got = elb.rmsnorm(x, w, 1e-6)
        for i in range(3):
            want = ol.rmsnorm(x[i], w, 1e-6)
            assert np.abs(got[i] - want).max() <= 2e-7 * np.abs(want).max()


@pytest.mark.parametrize("t", (synth.Q8_0, synth.F16))
@pytest.mark.parametrize("b", (3, 64, 200))
def test_matmul_fp16_tensor_cores_long_rows(elb, t, b):
    """F16 and Q8_0 weights on the tcgen05 kind::f16 kernel with a long row (n = 6144: 24 accumulation segments, k splits
    when the batch has few tiles): against float64 on the decoded weights the result must be as good as the CPU path's to
    within 2e-6 of the largest output (a single tensor-memory chain over all of k was 3e-5 off), and twice the same bits."""
    rng = np.random.default_rng(7 * b + t)
    rows, n = 384, 6144
    wb = synth.rand_weight(rng, t, rows, n)
    x = (rng.normal(size=(b, n)) + 0.5).astype(np.float32)  # a non-zero mean: long sums of one sign
    w = elb.Weight(t, rows, n, wb, planes=True)
    y = w.matmul(x, 4)
    deq = ol.dequant_rows(t, rows, n, wb).astype(np.float64)
    exact = x.astype(np.float64) @ deq.T
    scale = np.abs(exact).max(axis=1, keepdims=True)
    e_gpu = float((np.abs(y - exact) / scale).max())
    ref = np.stack([ol.matvec(t, rows, n, wb, x[i]) for i in range(0, b, max(1, b // 8))])
    e_cpu = float((np.abs(ref - exact[::max(1, b // 8)]) / scale[::max(1, b // 8)]).max())
    print(f"\ntype {t} b {b}: relative error against float64: gpu {e_gpu:.2e}, cpu path {e_cpu:.2e}")
    assert e_gpu <= e_cpu + 2e-6, (e_gpu, e_cpu)
    assert np.array_equal(bits(y), bits(w.matmul(x, 4))), "matmul must be deterministic"


def test_bounded_wait_expiry_is_reported(elb):
    """The failure path of the device-side waits, made on the host: a barrier that nobody arrives at. The kernel's
    bounded wait must give up and raise the error word; the library reports ELB_ERR_CUDA, and the device stays usable."""
    from exactinfer_b200 import capi
    rc = capi.lib().elb_selftest_wait_expiry(0)
    assert rc == capi.ERR_CUDA, rc
    assert b"wait" in capi.lib().elb_last_error()
    assert capi.lib().elb_selftest_wait_expiry(0) == capi.ERR_CUDA  # the error word was cleared and is raised again
    rng = np.random.default_rng(3)
    wb = synth.rand_weight(rng, synth.F16, 64, 256)
    x = rng.normal(size=(20, 256)).astype(np.float32)
    w = elb.Weight(synth.F16, 64, 256, wb)
    y = w.matmul(x, 4)  # the same kernel family, after the expiry
    for i in (0, 19):
        check_matvec(y[i], wb, synth.F16, 64, 256, x[i])


@pytest.mark.parametrize("t", (synth.Q4_K, synth.Q6_K))
@pytest.mark.parametrize("b,nl", ((24, 4), (70, 3), (200, 4)))
def test_matmul_accumulator_columns_bit_exact(elb, t, b, nl):
    """The int32 accumulators of the tcgen05 limb GEMM as they leave tensor memory, joined over their columns, are the
    block sums of the limb products: sum_c 256^c A[token][block][c][row] == sum_l 256^l I[row][block][l] with I from the
    oracle's integer path, for every token, row and 256-block, exactly (no tolerance: these are integers)."""
    rng = np.random.default_rng(11 * b + t)
    rows, n = 200, 1024
    wb = synth.rand_weight(rng, t, rows, n)
    x = rng.normal(size=(b, n)).astype(np.float32)
    x[1] *= 300.0
    w = elb.Weight(t, rows, n, wb, planes=True)
    A = w.matmul_acc(x, nl).astype(np.int64)  # [b][nblk][nl + 1][rows]
    got = sum(A[:, :, c, :] << (8 * c) for c in range(nl + 1))  # [b][nblk][rows]
    assert np.abs(A).max() < 2 ** 23, "a column must stay below the bound the join relies on"
    for i in range(b):
        limbs, _, _ = ol.split_limbs(x[i], nl)
        I, _ = ol.limb_block_sums(t, rows, n, wb, limbs)  # [rows][nblk][nl]
        want = sum(I[:, :, l].astype(np.int64) << (8 * l) for l in range(nl))
        assert np.array_equal(got[i], want.T), f"token {i}"
    w.close()
