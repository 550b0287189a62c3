"""GPU parity tests of the attention path: the row softmax (reference signature
src/cuda_kernels/sm120_c_interface.h:189-195 and the masked form), the fused
tcgen05 attention kernel (reference signature :138-144) and the unfused route,
and the SM120MultiHeadAttention layer, against the float64 oracle."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu

DT = {"float32": 0, "float16": 1, "bfloat16": 2}
SOFTMAX_TOL = {"float32": 2e-6, "float16": 6e-4, "bfloat16": 5e-3}      # absolute, on probabilities in [0, 1]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_softmax_rows(ops, binding, dtype):
    rng = np.random.default_rng(1)
    for rows, cols in ((1, 1), (3, 7), (5, 64), (33, 1000), (64, 2048), (9, 8192), (4, 10000), (2, 3)):
        x = ref.quantize(4.0 * rng.standard_normal((rows, cols), dtype=np.float32), dtype)
        got = ops.softmax(U.to_cuda(x))
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == "softmax_rows"
        want = ref.softmax_oracle(x)
        g = U.to_numpy(got).astype(np.float64)
        assert np.max(np.abs(g - want)) <= SOFTMAX_TOL[dtype], (rows, cols)
        assert np.max(np.abs(g.sum(-1) - 1.0)) <= 200 * SOFTMAX_TOL[dtype]


def test_softmax_other_axes_and_reference_signature(ops, binding):
    lib = binding.load_library()
    rng = np.random.default_rng(2)
    x = rng.standard_normal((6, 50, 12), dtype=np.float32)
    tx = torch.from_numpy(x).cuda()
    for axis in (0, 1, 2, -2):
        got = ops.softmax(tx, axis=axis).cpu().numpy()
        assert np.max(np.abs(got - ref.softmax_oracle(x, axis=axis))) <= 2e-6, axis
    # sm120_launch_softmax(logits, output, outer, axis, inner, dtype, stream), in place, half
    h = torch.from_numpy(x).cuda().half()
    want = ref.softmax_oracle(U.to_numpy(h), axis=1)
    assert lib.sm120_launch_softmax(h.data_ptr(), h.data_ptr(), 6, 50, 12, 1, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert np.max(np.abs(U.to_numpy(h).astype(np.float64) - want)) <= 6e-4
    assert lib.sm120_launch_softmax(h.data_ptr(), h.data_ptr(), 6, 50, 12, 3, None) == 1          # FP8: rejected
    assert lib.sm120_launch_softmax(h.data_ptr(), h.data_ptr(), -1, 50, 12, 1, None) == 1
    assert lib.sm120_launch_softmax(None, None, 0, 50, 12, 1, None) == 0


def test_softmax_scale_mask_causal(binding):
    lib = binding.load_library()
    rng = np.random.default_rng(3)
    bh, sq, sk = 3, 40, 72
    x = rng.standard_normal((bh * sq, sk), dtype=np.float32)
    mask = (rng.random((sq, sk)) < 0.3).astype(np.float32)
    tx, tm = torch.from_numpy(x).cuda(), torch.from_numpy(mask).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    for out_dt, tol in (("float32", 2e-6), ("bfloat16", 5e-3)):
        out = torch.empty(bh * sq, sk, device="cuda", dtype=U.torch_dtype(out_dt))
        rc = lib.sm120_launch_softmax_ex(tx.data_ptr(), out.data_ptr(), bh * sq, sk, 0, DT[out_dt], 0.25, tm.data_ptr(), sq, -1e9, 1, sq, stream)
        assert rc == 0
        torch.cuda.synchronize()
        s = x.astype(np.float64).reshape(bh, sq, sk) * 0.25 + mask.astype(np.float64) * -1e9
        keep = np.arange(sk)[None, :] <= (np.arange(sq)[:, None] + sk - sq)
        want = ref.softmax_oracle(np.where(keep, s, -np.inf)).reshape(bh * sq, sk)
        assert np.max(np.abs(U.to_numpy(out).astype(np.float64) - want)) <= tol, out_dt
    # argument checks: mask with a strided axis, causal with more queries than keys, fp16 -> fp32
    assert lib.sm120_launch_softmax_ex(tx.data_ptr(), tx.data_ptr(), 10, sk, 0, 0, 1.0, None, 0, 0.0, 1, 100, stream) == 1
    assert lib.sm120_launch_softmax_ex(tx.data_ptr(), tx.data_ptr(), 10, sk, 1, 0, 1.0, None, 0, 0.0, 0, 0, stream) == 1


def _qkv(rng, lead, sq, sk, d, dtype, spread=1.0):
    q = ref.quantize(spread * rng.standard_normal(lead + (sq, d), dtype=np.float32), dtype)
    k = ref.quantize(spread * rng.standard_normal(lead + (sk, d), dtype=np.float32), dtype)
    v = ref.quantize(rng.standard_normal(lead + (sk, d), dtype=np.float32), dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("d", [64, 128])
def test_fused_attention_matches_oracle(ops, binding, dtype, d):
    rng = np.random.default_rng(10 + d)
    for lead, sq, sk, causal in (((2, 3), 128, 128, False), ((1, 2), 256, 384, False), ((2,), 200, 200, False),
                                 ((3,), 1000, 1000, True), ((1, 1), 130, 700, True), ((2,), 1, 257, False), ((1,), 512, 512, True)):
        q, k, v = _qkv(rng, lead, sq, sk, d, dtype)
        got = ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k), U.to_cuda(v), causal_mask=causal)
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == f"attention_tcgen05_d{d}", binding.last_kernel_name()
        want = ref.attention_oracle(q, k, v, causal=causal)
        g = U.to_numpy(got)
        assert g.shape == want.shape and np.isfinite(g.astype(np.float32)).all()
        err = ref.rel_frobenius(g, want)
        assert err <= ref.TOLERANCE[dtype], (lead, sq, sk, causal, err)
    # a sharper softmax (larger scores) and an explicit scale
    q, k, v = _qkv(rng, (2, 2), 256, 256, d, dtype, spread=2.0)
    got = ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k), U.to_cuda(v), scale=0.3)
    assert ref.rel_frobenius(U.to_numpy(got), ref.attention_oracle(q, k, v, scale=0.3)) <= ref.TOLERANCE[dtype]
    # run-to-run identical
    again = ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k), U.to_cuda(v), scale=0.3)
    assert torch.equal(got, again)
    st = ctypes.c_uint(1)
    assert binding.load_library().sm120_get_kernel_status(0, ctypes.byref(st), 0) == 0 and st.value == 0


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("d", [64, 128])
def test_fused_attention_growing_scores_and_scale_signs(ops, binding, dtype, d):
    """Keys whose scores grow from tile to tile move the kernel's reference maximum again and again (it rescales
    its accumulator in tensor memory, one group of key tiles independently of the other, and merges the two at the
    end); a negative scale turns the maximum search into a minimum search; scale 0 is the plain mean of V."""
    rng = np.random.default_rng(40 + d)
    lead, sq, sk = (2,), 200, 1100                      # nine key tiles, the last one ragged
    q, k, v = _qkv(rng, lead, sq, sk, d, dtype)
    grow = (1.0 + 0.75 * (np.arange(sk) // 128)).astype(np.float32)[:, None]     # tile t: scores x (1 + 0.75 t)
    k = ref.quantize(k.astype(np.float32) * grow, dtype)
    for scale, causal in ((1.0, False), (1.0, True), (-1.0, False), (-0.7, True), (0.0, False)):
        cq = q if not causal else ref.quantize(np.concatenate([q] * 6, axis=-2)[..., :sk, :], dtype)
        got = ops.scaled_dot_product_attention(U.to_cuda(cq), U.to_cuda(k), U.to_cuda(v), scale=scale, causal_mask=causal)
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == f"attention_tcgen05_d{d}"
        want = ref.attention_oracle(cq, k, v, scale=scale, causal=causal)
        g = U.to_numpy(got)
        assert np.isfinite(g.astype(np.float32)).all()
        err = ref.rel_frobenius(g, want)
        assert err <= ref.TOLERANCE[dtype], (scale, causal, err)
    # scores that SHRINK from tile to tile: the reference maximum of the first tiles stays, nothing is rescaled
    k2 = ref.quantize(k.astype(np.float32)[..., ::-1, :].copy(), dtype)
    got = ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k2), U.to_cuda(v), scale=1.0)
    assert ref.rel_frobenius(U.to_numpy(got), ref.attention_oracle(q, k2, v, scale=1.0)) <= ref.TOLERANCE[dtype]
    st = ctypes.c_uint(1)
    assert binding.load_library().sm120_get_kernel_status(0, ctypes.byref(st), 0) == 0 and st.value == 0


def test_attention_reference_signature_and_weights(binding):
    # sm120_launch_attention(queries, keys, values, output, attention_weights, batch, seq_len, head_dim, scale, dtype, stream)
    lib = binding.load_library()
    rng = np.random.default_rng(20)
    stream = torch.cuda.current_stream().cuda_stream
    bh, s, d = 4, 192, 64
    for dtype in ("float16", "float32"):
        q, k, v = _qkv(rng, (bh,), s, s, d, dtype)
        tq, tk, tv = U.to_cuda(q), U.to_cuda(k), U.to_cuda(v)
        out = torch.empty_like(tq)
        w = torch.empty(bh, s, s, device="cuda")
        assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), w.data_ptr(), bh, s, d,
                                          0.125, DT[dtype], stream) == 0
        torch.cuda.synchronize()
        want, want_w = ref.attention_oracle(q, k, v, scale=0.125, return_weights=True)
        assert ref.rel_frobenius(U.to_numpy(out), want) <= ref.TOLERANCE[dtype] * (10 if dtype == "float32" else 1)
        assert np.max(np.abs(w.cpu().numpy() - want_w)) <= (2e-5 if dtype == "float32" else 2e-3)
        if dtype == "float16":      # no weights requested: the fused kernel alone, same output
            out2 = torch.empty_like(tq)
            assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out2.data_ptr(), None, bh, s, d, 0.125, 1, stream) == 0
            assert torch.equal(out, out2)
        else:                       # fp32 needs the weights buffer as its score matrix
            assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), None, bh, s, d, 0.125, 0, stream) == 1
    # a head size the fused kernel lacks, FP8, negative sizes: rejected before any launch
    assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), None, bh, s, 48, 0.1, 1, stream) == 1
    assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), None, bh, s, d, 0.1, 3, stream) == 1
    assert lib.sm120_launch_attention(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), None, -1, s, d, 0.1, 1, stream) == 1
    assert lib.sm120_launch_attention(None, None, None, None, None, 0, s, d, 0.1, 1, stream) == 0
    torch.cuda.synchronize()


def test_unfused_attention_with_mask_and_flash_signature(ops, binding):
    rng = np.random.default_rng(30)
    lead, sq, sk, d = (2, 2), 96, 160, 64
    q, k, v = _qkv(rng, lead, sq, sk, d, "bfloat16")
    mask = (rng.random((sq, sk)) < 0.25).astype(np.float32)
    tq, tk, tv = U.to_cuda(q), U.to_cuda(k), U.to_cuda(v)
    got, w = ops.scaled_dot_product_attention(tq, tk, tv, attention_mask=torch.from_numpy(mask).cuda(), return_attention_scores=True)
    want, want_w = ref.attention_oracle(q, k, v, mask=mask, return_weights=True)
    assert ref.rel_frobenius(U.to_numpy(got), want) <= ref.TOLERANCE["bfloat16"]
    assert np.max(np.abs(w.cpu().numpy() - want_w)) <= 5e-3
    # per-batch masks
    mask4 = (rng.random(lead + (sq, sk)) < 0.25).astype(np.float32)
    got = ops.scaled_dot_product_attention(tq, tk, tv, attention_mask=torch.from_numpy(mask4).cuda())
    assert ref.rel_frobenius(U.to_numpy(got), ref.attention_oracle(q, k, v, mask=mask4)) <= ref.TOLERANCE["bfloat16"]
    # fp32 tensors, a head size without a fused kernel
    q32, k32, v32 = _qkv(rng, (3,), 70, 90, 48, "float32")
    got = ops.scaled_dot_product_attention(U.to_cuda(q32), U.to_cuda(k32), U.to_cuda(v32), causal_mask=True)
    assert ref.rel_frobenius(U.to_numpy(got), ref.attention_oracle(q32, k32, v32, causal=True)) <= 1e-4
    # flash_attention: 4-D tensors, additive mask, returns (output, weights)
    add = np.where(mask > 0, -1e9, 0.0).astype(np.float32)
    out, w = ops.flash_attention(tq, tk, tv, attention_mask=torch.from_numpy(add).cuda(), causal_mask=False)
    assert ref.rel_frobenius(U.to_numpy(out), want) <= ref.TOLERANCE["bfloat16"]
    assert tuple(w.shape) == lead + (sq, sk)
    with pytest.raises(ValueError):
        ops.flash_attention(tq[0], tk[0], tv[0])
    with pytest.raises(NotImplementedError):
        ops.scaled_dot_product_attention(tq, tk, tv, dropout_rate=0.1)


def test_multi_head_attention_layer(pkg):
    layers = pkg.sm120_keras_layers
    torch.manual_seed(5)
    batch, seq, dim, heads, key_dim = 3, 144, 256, 4, 64
    layer = layers.SM120MultiHeadAttention(heads, key_dim, dtype="bfloat16")
    x = torch.randn(batch, seq, dim, device="cuda").bfloat16()
    layer.build(tuple(x.shape), seed=11)
    y = layer(x)
    assert tuple(y.shape) == (batch, seq, dim) and y.dtype == torch.bfloat16 and len(layer.weights) == 8
    # the same computation in float64 from the layer's own weights
    f = lambda t: U.to_numpy(t).astype(np.float64)
    xd = f(x)
    proj = lambda dense, inp: inp @ f(dense.kernel) + f(dense.bias)
    split = lambda t: t.reshape(batch, seq, heads, key_dim).transpose(0, 2, 1, 3)
    q, k, v = (split(proj(dn, xd)) for dn in (layer.query_dense, layer.key_dense, layer.value_dense))
    att = ref.attention_oracle(q, k, v).transpose(0, 2, 1, 3).reshape(batch, seq, heads * key_dim)
    want = proj(layer.output_dense, att)
    assert ref.rel_frobenius(U.to_numpy(y), want) <= 2e-2           # four 16-bit roundings of intermediate tensors
    # cross attention from a list, with the attention weights
    mem = torch.randn(batch, 80, dim, device="cuda").bfloat16()
    y2, w = layer([x, mem, mem], return_attention_scores=True)
    assert tuple(y2.shape) == (batch, seq, dim) and tuple(w.shape) == (batch, heads, seq, 80)
    assert float((w.sum(-1) - 1).abs().max()) <= 1e-3
    cfg = layer.get_config()
    assert cfg["num_heads"] == heads and cfg["key_dim"] == key_dim and cfg["use_flash_attention"] is True
    assert layers.get_custom_objects()["SM120MultiHeadAttention"] is layers.SM120MultiHeadAttention


def test_attention_full_size_attention_score_shape(ops, binding):
    """Batch 64 of [2048 x 128] queries and keys (the batched attention-score benchmark shape) through the fused
    kernel: sampled query rows against the float64 oracle, and determinism."""
    torch.manual_seed(3)
    bh, s, d = 64, 2048, 128
    q = torch.randn(bh, s, d, device="cuda").bfloat16()
    k = torch.randn(bh, s, d, device="cuda").bfloat16()
    v = torch.randn(bh, s, d, device="cuda").bfloat16()
    out = ops.scaled_dot_product_attention(q, k, v)
    assert binding.last_kernel_name() == "attention_tcgen05_d128"
    for b in (0, 17, 63):
        rows = torch.randint(0, s, (24,), device="cuda")
        want = ref.attention_oracle(U.to_numpy(q[b][rows]), U.to_numpy(k[b]), U.to_numpy(v[b]))
        assert ref.rel_frobenius(U.to_numpy(out[b][rows]), want) <= ref.TOLERANCE["bfloat16"], b
    assert torch.equal(ops.scaled_dot_product_attention(q, k, v), out)
    # the unfused route (GEMM, softmax, GEMM) agrees with the fused kernel
    two = ops.scaled_dot_product_attention(q[:4], k[:4], v[:4], attention_mask=torch.zeros(s, s, device="cuda"))
    assert ref.rel_frobenius(U.to_numpy(two), U.to_numpy(out[:4]).astype(np.float64)) <= ref.TOLERANCE["bfloat16"]


_ATT_SWEEP_LENS = [1, 5, 64, 127, 128, 129, 200, 256, 383, 512, 700, 1024, 1300]


@pytest.mark.parametrize("seed", range(32))
def test_fused_attention_seeded_sweep(ops, binding, seed):
    """Batch shape, query and key counts (ragged, shorter and longer than one tile, more queries than keys), head size,
    type, scale, score spread and the causal switch drawn together from one seeded stream.  Causal attention with
    more queries than keys is an argument error; the case then runs without the causal switch."""
    rng = np.random.default_rng(7000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    dtype, d = pick(["bfloat16", "float16"]), pick([64, 128])
    lead = pick([(1,), (3,), (2, 2), (1, 5)])
    sq, sk = pick(_ATT_SWEEP_LENS), pick(_ATT_SWEEP_LENS)
    causal = bool(rng.integers(2))
    scale = pick([None, None, 0.05, 0.2, -0.1])
    q, k, v = _qkv(rng, lead, sq, sk, d, dtype, spread=pick([0.5, 1.0, 2.0]))
    what = (dtype, d, lead, sq, sk, causal, scale)
    if causal and sq > sk:                     # queries with no key to look at: rejected, not computed
        with pytest.raises(ops.InvalidArgumentError):
            ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k), U.to_cuda(v), scale=scale, causal_mask=True)
        causal = False
    got = ops.scaled_dot_product_attention(U.to_cuda(q), U.to_cuda(k), U.to_cuda(v), scale=scale, causal_mask=causal)
    torch.cuda.synchronize()
    assert binding.last_kernel_name() == f"attention_tcgen05_d{d}", what
    want = ref.attention_oracle(q, k, v, scale=scale, causal=causal)
    g = U.to_numpy(got)
    assert g.shape == want.shape and np.isfinite(g.astype(np.float32)).all(), what
    err = ref.rel_frobenius(g, want)
    assert err <= ref.TOLERANCE[dtype], what + (err,)
