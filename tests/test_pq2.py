"""PQ2_0 ternary rows: the oracle pinned to the reference's known answers (CPU), and the CUDA
matvec, through the C ABI, against the oracle (GPU).

Bar for the product (floating point): |y - y_oracle| <= 2e-5 * sum_j |x_j| |w_j| per output.  The
reference ships three summation orders for this product (decoded-row dot, scalar block dot, AVX2)
and bounds their mutual difference by 1e-4 relative in its own test (src/kernels.rs:855-906);
the norm-wise form used here is the same bound without the blow-up on outputs that cancel to ~0.
"""
import numpy as np
import pytest

TOL = 2e-5


def synth(bk, seed, n_rows, ne0, n_tok, x_scale=1.0):
    rng = np.random.default_rng(seed)
    nb = -(-ne0 // 128)
    codes = rng.integers(0, 4, size=(n_rows, ne0), dtype=np.uint8)
    scales = (0.01 + rng.random((n_rows, nb)) * 2.0).astype(np.float16)
    payload = bk.pack_pq2(codes, scales)
    x = (rng.standard_normal((n_tok, ne0)) * x_scale).astype(np.float32)
    return payload, codes, scales, x


def dense(codes, scales, ne0):
    w = codes.astype(np.float64) - 1.0
    return w * np.repeat(scales.astype(np.float64), 128, axis=1)[:, :ne0]


# ---- CPU: the oracle against the reference's own tests -------------------------------------------

def test_pq2_decode_known_row(oracle):
    # src/kernels.rs:774-787: scale 0x4000 = 2.0; code 3 at j = 0, code 1 at j = 4, code 2 at j = 5
    raw = np.zeros(34, np.uint8)
    raw[1] = 0x40
    raw[2] = 0b11
    raw[3] = 0b1001
    v = oracle.pq2_decode_row(raw, 128)
    assert v[0] == 4.0 and v[1] == -2.0 and v[4] == 0.0 and v[5] == 2.0
    assert v.size == 128 and np.all(v[6:] == -2.0)


def test_pq2_row_bytes(oracle, bk):
    for ne0, want in ((128, 34), (129, 68), (256, 68), (5120, 1360), (6144, 1632), (1, 34)):
        assert oracle.pq2_row_bytes(ne0) == want == bk.pq2_row_bytes(ne0)


def test_pq2_matmul_n_matches_per_token_matvec(oracle, bk):
    # src/kernels.rs:909-947: the N-column product equals the per-token matvec exactly
    payload, _, _, x = synth(bk, 1, 12, 256, 3)
    y_n = oracle.pq2_matmul(payload, 256, 0, 12, x, 3)
    for t in range(3):
        assert np.array_equal(y_n[t], oracle.pq2_matmul(payload, 256, 0, 12, x[t], 1)[0])


def test_pq2_scalar_dot_matches_decoded_dot_and_f64(oracle, bk):
    ne0, n_rows = 5120, 8  # the model's row width (src/kernels.rs:864)
    payload, codes, scales, x = synth(bk, 2, n_rows, ne0, 1)
    w = dense(codes, scales, ne0)
    y = oracle.pq2_matmul(payload, ne0, 0, n_rows, x, 1)[0]
    norm = np.abs(w) @ np.abs(x[0].astype(np.float64))
    truth = w @ x[0].astype(np.float64)
    assert np.all(np.abs(y - truth) <= TOL * norm)
    for r in range(n_rows):
        assert abs(oracle.pq2_dot_row(payload, ne0, r, x[0]) - y[r]) <= TOL * norm[r]
        assert np.array_equal(oracle.pq2_decode_row(payload[r * 1360:(r + 1) * 1360], ne0), w[r].astype(np.float32))


def test_pq2_ragged_row_ignores_codes_past_ne0(oracle, bk):
    ne0 = 200
    payload, codes, scales, x = synth(bk, 3, 5, ne0, 1)
    dirty = payload.copy().reshape(5, 2, 34)
    dirty[:, 1, 2 + (ne0 - 128) // 4:] = 0xFF  # codes past ne0 in the last block
    y0 = oracle.pq2_matmul(payload, ne0, 0, 5, x, 1)
    y1 = oracle.pq2_matmul(dirty.reshape(-1), ne0, 0, 5, x, 1)
    assert np.array_equal(y0, y1)
    assert oracle.pq2_decode_row(payload[:68], ne0).size == ne0


def test_pq2_range_errors(oracle, bk):
    payload, _, _, x = synth(bk, 4, 4, 128, 1)
    with pytest.raises(ValueError):
        oracle.pq2_matmul(payload, 128, 2, 3, x, 1)  # rows 2..5 of 4 (src/kernels.rs:288-299)
    with pytest.raises(ValueError):
        oracle.pq2_matmul(payload, 128, 0, 4, x[0, :100], 1)  # x length (src/kernels.rs:282-284)
    with pytest.raises(ValueError):
        oracle.pq2_dot_row(payload, 128, 4, x[0])


# ---- GPU: the CUDA matvec against the oracle -------------------------------------------------------

SHAPES = [(5120, 1024, 1), (5120, 1000, 1), (6144, 512, 1), (256, 12, 3), (200, 37, 2), (5120, 64, 4), (5120, 33, 7),
          (128, 1, 1), (17408, 48, 1), (5120, 16 * 300, 2)]


@pytest.mark.gpu
@pytest.mark.parametrize("ne0,n_rows,n_tok", SHAPES)
def test_gpu_pq2_matvec_matches_oracle(oracle, bk, gpu_ctx, ne0, n_rows, n_tok):
    payload, codes, scales, x = synth(bk, ne0 + n_rows + n_tok, n_rows, ne0, n_tok)
    t = bk.Pq2Tensor(gpu_ctx, payload, ne0)
    got = t.matmul_n(x, n_tok)
    gpu_ctx.synchronize()
    want = oracle.pq2_matmul(payload, ne0, 0, n_rows, x, n_tok)
    w = dense(codes, scales, ne0)
    norm = np.abs(x.astype(np.float64)) @ np.abs(w).T
    truth = x.astype(np.float64) @ w.T
    assert np.all(np.abs(got - want) <= TOL * norm + 1e-30), f"max {np.max(np.abs(got - want) / (norm + 1e-30)):.3e}"
    assert np.max(np.abs(got - truth) / (norm + 1e-30)) <= 2e-6  # exact block sums of 25-bit fixed-point x, f32 sums across blocks
    t.free()


@pytest.mark.gpu
def test_gpu_pq2_row_ranges_aligned_and_not(oracle, bk, gpu_ctx):
    # ne0 = 128: rows of 34 bytes, so most base rows start off a 16-byte boundary (plain-load path)
    for ne0, n_all in ((128, 70), (5120, 90)):
        payload, _, _, x = synth(bk, 11 + ne0, n_all, ne0, 1)
        t = bk.Pq2Tensor(gpu_ctx, payload, ne0)
        for base, n in ((0, n_all), (3, 40), (8, 33), (16, 16), (n_all - 1, 1), (5, 0)):
            got = t.matvec(x[0], base_row=base, n_rows=n)
            want = oracle.pq2_matmul(payload, ne0, base, n, x, 1)[0]
            full = oracle.pq2_matmul(payload, ne0, 0, n_all, x, 1)[0]
            assert np.array_equal(want, full[base:base + n])
            assert np.all(np.abs(got - want) <= TOL * np.abs(x[0]).sum() * 2.0)
        t.free()


@pytest.mark.gpu
def test_gpu_pq2_errors_like_the_reference(bk, gpu_ctx):
    payload, _, _, x = synth(bk, 5, 4, 128, 1)
    t = bk.Pq2Tensor(gpu_ctx, payload, 128)
    with pytest.raises(bk.BonsaiKvError) as e:
        t.matvec(x[0], base_row=2, n_rows=3)
    assert e.value.status == bk._abi.BK_ERR_RANGE and "payload is" in str(e.value)
    with pytest.raises(bk.BonsaiKvError):
        t.matvec(x[0, :100])
    t.free()


@pytest.mark.gpu
def test_gpu_pq2_properties_at_model_size(bk, gpu_ctx):
    """wq of a full-attention layer (12288 x 5120): exact behaviour that needs no oracle."""
    ne0, n_rows = 5120, 12288
    rng = np.random.default_rng(99)
    nb = ne0 // 128
    x = rng.standard_normal((1, ne0)).astype(np.float32)
    # weight 0 everywhere (code 1): exactly zero; weight +1 with scale 1 (code 2): the sum of x
    zeros = bk.Pq2Tensor(gpu_ctx, bk.pack_pq2(np.ones((64, ne0), np.uint8), np.ones((64, nb))), ne0)
    assert np.all(np.abs(zeros.matvec(x[0])) <= 1e-6 * np.abs(x).sum())
    ones = bk.Pq2Tensor(gpu_ctx, bk.pack_pq2(np.full((64, ne0), 2, np.uint8), np.ones((64, nb))), ne0)
    assert np.allclose(ones.matvec(x[0]), x.astype(np.float64).sum(), rtol=0, atol=2e-6 * np.abs(x).sum())
    zeros.free()
    ones.free()
    codes = rng.integers(0, 4, size=(n_rows, ne0), dtype=np.uint8)
    scales = (0.01 + rng.random((n_rows, nb))).astype(np.float16)
    t = bk.Pq2Tensor(gpu_ctx, bk.pack_pq2(codes, scales), ne0)
    y = t.matvec(x[0])
    # a power-of-two factor on x passes through exactly (the kernel normalises every block of x by a power of two)
    assert np.array_equal(t.matvec(x[0] * np.float32(1024.0)), y * np.float32(1024.0))
    assert np.array_equal(t.matvec(x[0] * np.float32(2.0 ** -20)), y * np.float32(2.0 ** -20))
    # rows are independent: any row range equals the slice of the whole product
    assert np.array_equal(t.matvec(x[0], base_row=4096, n_rows=1024), y[4096:5120])
    # against float64 on a sample of rows
    rows = rng.choice(n_rows, 64, replace=False)
    w = dense(codes[rows], scales[rows], ne0)
    assert np.max(np.abs(y[rows] - w @ x[0].astype(np.float64)) / (np.abs(w) @ np.abs(x[0]).astype(np.float64))) <= 2e-6
    t.free()


@pytest.mark.gpu
def test_gpu_pq2_multi_equals_separate_calls(bk, gpu_ctx):
    """attn_q, attn_k, attn_v shapes on one x in one launch: bit-equal to three launches."""
    ne0 = 5120
    rng = np.random.default_rng(7)
    tensors = []
    for n_rows in (12288, 1024, 1000):
        payload, _, _, _ = synth(bk, n_rows, n_rows, ne0, 1)
        tensors.append(bk.Pq2Tensor(gpu_ctx, payload, ne0))
    for n_tok in (1, 2, 3):
        x = rng.standard_normal((n_tok, ne0)).astype(np.float32)
        dx = gpu_ctx.to_device(x)
        ys = [gpu_ctx.alloc(n_tok * t.n_rows * 4) for t in tensors]
        bk.pq2_matvec_multi_device(gpu_ctx, tensors, dx.ptr, [y.ptr for y in ys], n_tok)
        for t, y in zip(tensors, ys):
            got = y.download((n_tok, t.n_rows), np.float32)
            assert np.array_equal(got, t.matmul_n(x, n_tok))
            y.free()
        dx.free()
    for t in tensors:
        t.free()
