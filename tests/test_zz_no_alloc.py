"""hm_gemv_bf16_noalloc: the projection kernel for callers that are not allowed to allocate.

Who that is: a host that runs kernels the way a pre-planned executor does -- every buffer is
owned and sized up front, kernels get pointers and nothing else -- or a serving loop that cannot
take the device-wide synchronisation and unpredictable latency an allocation may cost in the
middle of a token.  The ordinary entry point (hm_gemv_bf16) grows a cudaMalloc'd split-K scratch
on demand; this one keeps that scratch in an array compiled into the library, so it rejects
shapes that would need more than the array holds.

The test calls both entry points through the C ABI on the same device-resident inputs and
expects identical outputs (same kernel, same split, same reduction order), twice in a row and
across a larger-then-smaller shape so stale scratch contents would show.  The ordinary entry
point is switched to its global-scratch reduction (HM_NO_CLUSTER=1) for the comparison, since
that is the reduction the allocation-free variant uses; its default, the reduction through a
thread-block cluster, sums in a different order and is compared by tolerance.  The file is one
that pytest collects last."""
import numpy as np
import pytest

from homura_b200 import synth

pytestmark = pytest.mark.gpu


def _dev(hm, arr):
    b = hm.DeviceBuffer(arr.nbytes)
    b.upload(arr)
    return b


def _both(hm, x, w, M, K, N, layout):
    xd, wd = _dev(hm, x), _dev(hm, w)
    y_ref, y_new = hm.DeviceBuffer(M * N * 4), hm.DeviceBuffer(M * N * 4)
    y_new.upload(np.full(M * N, np.nan, np.float32))
    hm.gemv_bf16((xd.ptr, M), wd.ptr, layout, K=K, N=N, y=y_ref.ptr)
    hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, layout, M, K, N, y_new.ptr)
    hm.dev_sync()
    return y_ref.download(np.float32, M * N), y_new.download(np.float32, M * N)


def test_noalloc_matches_regular_entry_point_twice_in_a_row(hm, oracle, monkeypatch):
    monkeypatch.setenv("HM_NO_CLUSTER", "1")
    rng = np.random.default_rng(2024)
    # (M, K, N): split-K shapes of the decode step, a larger one, then a small one again
    shapes = [(1, 896, 1152), (1, 896, 1152), (8, 4864, 896), (16, 1536, 17920), (1, 896, 896), (4, 896, 9728)]
    for i, (M, K, N) in enumerate(shapes):
        w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
        x = rng.standard_normal((M, K), dtype=np.float32)
        for layout, wl in ((hm.LAYOUT_KN, w), (hm.LAYOUT_SLAB128, hm.pack_bf16_slabs(w))):
            ref, new = _both(hm, x, wl, M, K, N, layout)
            np.testing.assert_array_equal(new, ref)
            # and both are the right answer (tolerance of the kernel parity tests)
            want = oracle.matmul_bf16(x, w).ravel()
            assert np.abs(new - want).max() <= 2e-5 * np.abs(want).max()


def test_noalloc_agrees_with_cluster_reduction_within_tolerance(hm):
    rng = np.random.default_rng(77)
    M, K, N = 4, 4864, 896
    w = synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((M, K), dtype=np.float32)
    ref, new = _both(hm, x, hm.pack_bf16_slabs(w), M, K, N, hm.LAYOUT_SLAB128)
    assert np.abs(new - ref).max() <= 2e-5 * np.abs(ref).max()


def test_noalloc_rejects_what_it_cannot_serve(hm):
    x = np.zeros((1, 64), np.float32)
    w = np.zeros((64, 128), np.uint16)
    xd, wd, yd = _dev(hm, x), _dev(hm, w), hm.DeviceBuffer(128 * 4)
    with pytest.raises(hm.HomuraError) as e:  # host pointer: staging would need an allocation
        hm._check(hm.load_library().hm_gemv_bf16_noalloc(hm._ptr(x), hm._ptr(wd.ptr), hm.LAYOUT_KN, 1, 64, 128, hm._ptr(yd.ptr), None))
    assert e.value.status == hm.HM_ERR_INVALID and "device pointers" in e.value.message
    with pytest.raises(hm.HomuraError) as e:  # row count that would need a padded copy
        hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, hm.LAYOUT_KN, 3, 64, 128, yd.ptr)
    assert e.value.status == hm.HM_ERR_UNSUPPORTED
    with pytest.raises(hm.HomuraError) as e:  # more slabs than tickets: N > 524288
        hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, hm.LAYOUT_SLAB128, 1, 64, 128 * 4097, yd.ptr)
    assert e.value.status == hm.HM_ERR_UNSUPPORTED and "scratch" in e.value.message
    with pytest.raises(hm.HomuraError) as e:  # split-K partials beyond the built-in 4 MiB
        hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, hm.LAYOUT_SLAB128, 8, 16384, 128 * 600, yd.ptr)
    assert e.value.status == hm.HM_ERR_UNSUPPORTED


def test_noalloc_leaves_free_memory_unchanged(hm):
    # after one warm-up call (the first call on a device resolves the array's address and loads the kernels)
    # further calls must not move the device's free-memory figure
    rng = np.random.default_rng(5)
    M, K, N = 1, 4864, 896
    w = hm.pack_bf16_slabs(synth.f32_to_bf16_rne(rng.standard_normal((K, N), dtype=np.float32) * np.float32(0.02)))
    xd, wd, yd = _dev(hm, rng.standard_normal((M, K), dtype=np.float32)), _dev(hm, w), hm.DeviceBuffer(M * N * 4)
    hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, hm.LAYOUT_SLAB128, M, K, N, yd.ptr)
    hm.dev_sync()
    before = hm.dev_mem_info()[0]
    for _ in range(5):
        hm.gemv_bf16_noalloc(xd.ptr, wd.ptr, hm.LAYOUT_SLAB128, M, K, N, yd.ptr)
    hm.dev_sync()
    assert abs(hm.dev_mem_info()[0] - before) < (1 << 20)  # cudaMalloc hands out device memory in pieces of 2 MiB


def test_noalloc_rejects_buffers_of_another_gpu(hm):
    if hm.device_count() < 2:
        pytest.skip("needs two GPUs")
    x = np.zeros((1, 64), np.float32)
    w = np.zeros((64, 128), np.uint16)
    hm.dev_set(1)
    try:
        x1 = _dev(hm, x)  # lives on GPU 1
    finally:
        hm.dev_set(0)
    wd, yd = _dev(hm, w), hm.DeviceBuffer(128 * 4)
    with pytest.raises(hm.HomuraError) as e:  # the kernel on GPU 0 would read GPU 1's memory without peer access
        hm.gemv_bf16_noalloc(x1.ptr, wd.ptr, hm.LAYOUT_KN, 1, 64, 128, yd.ptr)
    assert e.value.status == hm.HM_ERR_INVALID and "current device" in e.value.message
    hm.dev_set(1)
    x1.free()
    hm.dev_set(0)
