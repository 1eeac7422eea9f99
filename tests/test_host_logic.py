"""CPU-only checks of the C ABI: the library loads, exports what include/dwbnq.h declares,
validates arguments like the reference does, derives quantizer parameters and the Pow2
threshold table correctly, and refuses to compute without a GPU (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _desc(L, **kw):
    base = dict(dtype=L.F32, c=8, n=2, h=16, w=16, kh=3, kw=3, stride_h=1, stride_w=1, pad_h=1, pad_w=1,
                dil_h=1, dil_w=1, multiplier=1)
    base.update(kw)
    return L.ConvDesc(**base)


def test_header_symbols_are_exported_and_bound(dwlib):
    text = "".join(open(os.path.join(ROOT, "include", h)).read()
                   for h in sorted(os.listdir(os.path.join(ROOT, "include"))) if h.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(dwbnq_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 20
    lib = dwlib.lib()
    for name in declared:
        assert hasattr(lib, name), "%s declared in include/*.h but not exported" % name
        assert name in dwlib.SIGNATURES, "%s has no ctypes signature" % name
    assert set(dwlib.SIGNATURES) == declared
    assert lib.dwbnq_version() == 1


def test_out_shape_and_validation(dwlib):
    lib = dwlib.lib()
    ho, wo = ctypes.c_int32(), ctypes.c_int32()
    cases = [((112, 112, 3, 1, 1, 1), (112, 112)), ((112, 112, 3, 2, 1, 1), (56, 56)),
             ((7, 7, 3, 1, 1, 1), (7, 7)), ((14, 14, 3, 2, 1, 1), (7, 7)), ((56, 56, 5, 1, 2, 1), (56, 56)),
             ((10, 9, 3, 2, 0, 2), (3, 3))]
    for (h, w, k, s, p, d), want in cases:
        desc = _desc(dwlib, h=h, w=w, kh=k, kw=k, stride_h=s, stride_w=s, pad_h=p, pad_w=p, dil_h=d, dil_w=d)
        assert lib.dwbnq_conv_out_shape(ctypes.byref(desc), ctypes.byref(ho), ctypes.byref(wo)) == dwlib.OK
        assert (ho.value, wo.value) == want
    bad = [dict(dtype=7), dict(c=0), dict(h=0), dict(kh=0), dict(stride_w=0), dict(pad_h=-1), dict(multiplier=0),
           dict(h=2, w=2, kh=5, kw=5, pad_h=0, pad_w=0)]
    for kw in bad:
        desc = _desc(dwlib, **kw)
        assert lib.dwbnq_conv_out_shape(ctypes.byref(desc), None, None) == dwlib.ERR_INVALID_ARG
        assert lib.dwbnq_last_error_string()
    assert lib.dwbnq_conv_out_shape(None, None, None) == dwlib.ERR_INVALID_ARG
    # the reference's limit: output-channels x filter-size <= 65536
    ok = _desc(dwlib, c=7281, kh=3, kw=3)
    assert lib.dwbnq_conv_out_shape(ctypes.byref(ok), None, None) == dwlib.OK
    over = _desc(dwlib, c=7282, kh=3, kw=3)
    assert lib.dwbnq_conv_out_shape(ctypes.byref(over), None, None) == dwlib.ERR_UNSUPPORTED
    assert b"65536" in lib.dwbnq_last_error_string()


def test_quantizer_parameters_match_oracle(dwlib, oracle):
    lib = dwlib.lib()
    a, b, c = ctypes.c_float(), ctypes.c_float(), ctypes.c_float()
    for sign in (0, 1):
        for n in (2, 4, 8, 16):
            for delta in (2.0 ** -4, 2.0 ** -3, 0.1, 1.0):
                assert lib.dwbnq_fpq_range(sign, n, delta, ctypes.byref(a), ctypes.byref(b)) == dwlib.OK
                assert (a.value, b.value) == oracle.fpq_params(sign, n, delta)
    assert lib.dwbnq_fpq_range(1, 1, 0.5, ctypes.byref(a), ctypes.byref(b)) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_fpq_range(0, 8, 0.0, ctypes.byref(a), ctypes.byref(b)) == dwlib.ERR_INVALID_ARG
    for sign in (0, 1):
        for wz in (0, 1):
            for n in (2, 4, 8, 10):
                for m in (-2, 0, 1, 3):
                    assert lib.dwbnq_pow2q_range(sign, wz, n, m, ctypes.byref(a), ctypes.byref(b),
                                                 ctypes.byref(c)) == dwlib.OK
                    assert (a.value, b.value, c.value) == oracle.pow2q_params(sign, wz, n, m)
    assert lib.dwbnq_workspace_bytes(192) >= 192 * 7 * 4 and lib.dwbnq_workspace_bytes(192) % 256 == 0
    assert lib.dwbnq_workspace_bytes(0) == 0


def _table_k(bits, table):
    """round(log2f(x)) for positive finite float bit patterns the way the device decides it."""
    bits = bits.astype(np.uint32)
    normal = bits >= 0x00800000
    e = np.where(normal, (bits >> 23).astype(np.int64) - 127, 0)
    sub = np.where(normal, 1, bits).astype(np.uint32)
    e_sub = np.floor(np.log2(sub.astype(np.float64))).astype(np.int64) - 149
    e = np.where(normal, e, e_sub)
    thr = table[e + 149]
    return (e + (bits >= thr)).astype(np.float32)


def test_pow2_threshold_table_reproduces_libm(dwlib, oracle):
    lib = dwlib.lib()
    table = np.zeros(277, np.uint32)
    assert lib.dwbnq_pow2q_threshold_table(table.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))) == dwlib.OK
    assert lib.dwbnq_pow2q_threshold_table(None) == dwlib.ERR_INVALID_ARG
    # the [1, 2) binade flips at the first float above sqrt(2)
    assert table[149] == 0x3fb504f4
    nthreads = oracle.max_threads()
    # every pattern within +-4096 of each binade's threshold, all denormals' binade edges
    chunks = []
    for e in range(-149, 128):
        lo = (e + 127) << 23 if e >= -126 else 1 << (e + 149)
        hi = lo + (1 << 23) if e >= -126 else 1 << (e + 150)
        t = int(table[e + 149])
        a, b = max(lo, t - 4096), min(hi, t + 4096)
        chunks.append(np.arange(a, b, dtype=np.uint32))
        chunks.append(np.arange(lo, min(hi, lo + 64), dtype=np.uint32))
        chunks.append(np.arange(max(lo, hi - 64), hi, dtype=np.uint32))
    rng = np.random.default_rng(0)
    chunks.append(rng.integers(1, 0x7f800000, size=1 << 24, dtype=np.uint32))
    bits = np.concatenate(chunks)
    want = oracle.round_log2(bits.view(np.float32), nthreads)
    np.testing.assert_array_equal(_table_k(bits, table), want)


def test_plan_selects_kernel_family(dwlib):
    lib = dwlib.lib()
    path, p, th, thr, smem = (ctypes.c_int() for _ in range(5))
    ctas = ctypes.c_int64()

    def plan(**kw):
        d = _desc(dwlib, **kw)
        st = lib.dwbnq_fused_plan(ctypes.byref(d), ctypes.c_void_p(4096), ctypes.c_void_p(8192), ctypes.byref(path),
                                  ctypes.byref(p), ctypes.byref(th), ctypes.byref(thr), ctypes.byref(ctas),
                                  ctypes.byref(smem))
        assert st == dwlib.OK, lib.dwbnq_last_error_string()
        return path.value

    for kw in (dict(dil_h=2, dil_w=2, pad_h=2, pad_w=2), dict(multiplier=2), dict(kh=7, kw=7, pad_h=3, pad_w=3),
               dict(pad_h=0, pad_w=0), dict(stride_h=3, stride_w=3), dict(h=1, kh=1, pad_h=0, stride_h=1)):
        assert plan(**kw) == dwlib.PATH_GENERIC
    for c, hw, s in ((32, 112, 1), (96, 112, 2), (144, 56, 1), (192, 28, 2), (384, 14, 1), (576, 14, 2), (960, 7, 1)):
        for dt in (dwlib.F32, dwlib.F16):
            assert plan(dtype=dt, n=4, c=c, h=hw, w=hw, stride_h=s, stride_w=s) in (dwlib.PATH_COOP, dwlib.PATH_TMA, dwlib.PATH_RAW, dwlib.PATH_PLANE, dwlib.PATH_PLANE_GEN)
            assert 1 <= thr.value <= 256  # one patch per thread
            assert smem.value <= 200 * 1024 and p.value >= 1 and th.value >= 1
            planes = 4 * c
            ho = (hw + 2 - 3) // s + 1
            assert ctas.value % (-(-planes // p.value)) == 0          # tiles = plane groups x row tiles
            assert (ctas.value // (-(-planes // p.value))) * th.value >= ho
    # which family serves which shape (3x3 / 5x5, pad k/2, aligned pointers)
    for hw, s, k in ((7, 1, 3), (14, 1, 3), (28, 1, 3), (56, 1, 3), (112, 1, 3), (14, 2, 3), (28, 2, 3), (56, 2, 3),
                     (112, 2, 3), (14, 1, 5), (56, 1, 5), (112, 1, 5)):
        assert plan(n=4, c=8, h=hw, w=hw, stride_h=s, stride_w=s, kh=k, kw=k, pad_h=k // 2, pad_w=k // 2) == dwlib.PATH_PLANE
        assert thr.value == 32 and smem.value <= 32 * 1024
    for hw in (6, 8, 10, 12, 16, 24, 30, 32):  # small planes, or a row pitch the TMA tile cannot take
        assert plan(n=4, c=8, h=hw, w=hw) == dwlib.PATH_PLANE_GEN, hw
    for hw in (40, 48, 80, 96):  # mid-size planes only the 8 x 8 blocks tile: the TMA tile where a driver offers it
        assert plan(n=4, c=8, h=hw, w=hw) in (dwlib.PATH_TMA, dwlib.PATH_PLANE_GEN), hw
    assert plan(n=4, c=8, h=42, w=42) == dwlib.PATH_PLANE_GEN   # 7 x 14 blocks tile it exactly
    assert plan(n=4, c=8, h=15, w=15) in (dwlib.PATH_RAW, dwlib.PATH_COOP)  # odd width
    assert plan(n=4, c=8, h=7, w=7, kh=5, kw=5, pad_h=2, pad_w=2) in (dwlib.PATH_RAW, dwlib.PATH_COOP)
    assert lib.dwbnq_set_forced_path(dwlib.PATH_GENERIC) == dwlib.OK
    assert plan(n=4, c=32, h=112, w=112) == dwlib.PATH_GENERIC
    assert lib.dwbnq_set_forced_path(dwlib.PATH_AUTO) == dwlib.OK
    assert lib.dwbnq_set_forced_path(9) == dwlib.ERR_INVALID_ARG


def test_argument_errors_before_any_cuda_call(dwlib):
    lib = dwlib.lib()
    d = _desc(dwlib)
    fake = ctypes.c_void_p(4096)
    assert lib.dwbnq_dwconv_fwd(ctypes.byref(d), None, fake, None, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_fpq_fwd(5, 16, 1, 8, 0.5, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_fpq_fwd(dwlib.F32, -1, 1, 8, 0.5, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_fpq_fwd(dwlib.F32, 16, 1, 8, -0.5, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_pow2q_fwd(dwlib.F32, 16, 1, 1, 0, 1, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_bn_infer_fwd(dwlib.F32, 2, 0, 4, 1e-5, fake, None, None, fake, fake, fake, -1,
                                  None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_bn_infer_fwd(dwlib.F32, 2, 3, 4, 1e-5, fake, None, None, None, fake, fake, -1,
                                  None) == dwlib.ERR_INVALID_ARG
    q = dwlib.QuantDesc(kind=dwlib.Q_MINMAX, x_min_max=1, eps=0.01)
    mm = dwlib.MinMaxPtrs(4096, 4096, 4096, 4096)
    # MinMax without a workspace / with a misaligned one
    assert lib.dwbnq_minmaxq_fwd(dwlib.F32, 2, 3, 4, ctypes.byref(q), fake, ctypes.byref(mm), fake, None, None, -1,
                                 None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_minmaxq_fwd(dwlib.F32, 2, 3, 4, ctypes.byref(q), fake, ctypes.byref(mm), fake,
                                 ctypes.c_void_p(4100), None, -1, None) == dwlib.ERR_INVALID_ARG
    qb = dwlib.QuantDesc(kind=9)
    assert lib.dwbnq_fused_fwd(ctypes.byref(d), 1e-5, ctypes.byref(qb), fake, fake, None, None, None, None, None,
                               None, fake, None, None, -1, None) == dwlib.ERR_INVALID_ARG
    # bn_mean without bn_var
    assert lib.dwbnq_fused_fwd(ctypes.byref(d), 1e-5, None, fake, fake, None, None, None, fake, None, None, fake,
                               None, None, -1, None) == dwlib.ERR_INVALID_ARG


def test_no_cpu_fallback_without_a_gpu(dwlib):
    lib = dwlib.lib()
    if lib.dwbnq_device_count() > 0:
        pytest.skip("a GPU is present; the refusal path is for GPU-less hosts")
    fake = ctypes.c_void_p(4096)
    st = lib.dwbnq_fpq_fwd(dwlib.F32, 16, 1, 8, 0.5, fake, fake, -1, None)
    assert st == dwlib.ERR_CUDA
    assert lib.dwbnq_last_error_string()
    d = _desc(dwlib)
    assert lib.dwbnq_dwconv_fwd(ctypes.byref(d), fake, fake, None, fake, -1, None) == dwlib.ERR_CUDA
    import torch
    from dwbnq import ops
    with pytest.raises(ValueError):
        ops.fixed_point_quantize(torch.zeros(4))


def test_planner_invariants_over_random_descriptors(dwlib):
    """Whatever the geometry, the planner answers OK with a launchable plan (or the reference's
    own limit error): shared memory below the 48 KB a launch gets without opting in for the
    one-warp families, one warp per CTA there, enough tiles to cover every plane and row."""
    lib = dwlib.lib()
    rng = np.random.default_rng(99)
    path, p, th, thr, smem = (ctypes.c_int() for _ in range(5))
    ctas = ctypes.c_int64()
    seen = set()
    for _ in range(3000):
        k = int(rng.choice([1, 3, 3, 3, 5, 7]))
        h, w = int(rng.integers(1, 130)), int(rng.integers(1, 130))
        if rng.random() < 0.5:
            w = h
        s = int(rng.choice([1, 1, 2, 3]))
        pad = int(rng.choice([0, k // 2, k // 2, k - 1]))
        dil = int(rng.choice([1, 1, 2]))
        mult = int(rng.choice([1, 1, 2]))
        n, c = int(rng.integers(1, 300)), int(rng.integers(1, 700))
        dt = int(rng.choice([dwlib.F32, dwlib.F16]))
        d = _desc(dwlib, dtype=dt, n=n, c=c, h=h, w=w, kh=k, kw=k, stride_h=s, stride_w=s, pad_h=pad, pad_w=pad,
                  dil_h=dil, dil_w=dil, multiplier=mult)
        al = int(rng.choice([0, 4]))  # aligned or 4 bytes off
        st = lib.dwbnq_fused_plan(ctypes.byref(d), ctypes.c_void_p(4096 + al), ctypes.c_void_p(8192 + al),
                                  ctypes.byref(path), ctypes.byref(p), ctypes.byref(th), ctypes.byref(thr),
                                  ctypes.byref(ctas), ctypes.byref(smem))
        fits = h + 2 * pad >= dil * (k - 1) + 1 and w + 2 * pad >= dil * (k - 1) + 1
        if not fits:
            assert st == dwlib.ERR_INVALID_ARG
            continue
        if c * mult * k * k > 65536:
            assert st == dwlib.ERR_UNSUPPORTED
            continue
        assert st == dwlib.OK, lib.dwbnq_last_error_string()
        seen.add(path.value)
        if path.value == dwlib.PATH_GENERIC:
            continue
        ho = (h + 2 * pad - dil * (k - 1) - 1) // s + 1
        assert p.value >= 1 and th.value >= 1 and ctas.value >= 1
        if path.value in (dwlib.PATH_PLANE, dwlib.PATH_PLANE_GEN):
            assert thr.value == 32 and smem.value <= 48 * 1024, (h, w, k, s, smem.value)
        else:
            assert 1 <= thr.value <= 256 and smem.value <= 200 * 1024
        assert k in (3, 5) and s in (1, 2) and pad == k // 2 and dil == 1 and mult == 1
        if path.value != dwlib.PATH_PLANE_GEN:  # (its bands run across plane boundaries)
            groups = -(-n * c // p.value)
            assert ctas.value % groups == 0 and (ctas.value // groups) * th.value >= ho, (h, w, k, s, path.value)
    assert {dwlib.PATH_GENERIC, dwlib.PATH_PLANE, dwlib.PATH_PLANE_GEN}.issubset(seen), seen


def test_pointwise_descriptor_validation_workspace_and_plan(dwlib):
    lib = dwlib.lib()
    P = dwlib.PwConvDesc
    good = P(dtype=dwlib.F32, c_in=32, c_out=96, h=14, w=14, n=4, math=dwlib.PW_MATH_FP32, act=dwlib.ACT_RELU6)
    # coefficients of the 96 channels (one tile of 96 columns) + the two TF32 halves of w
    assert lib.dwbnq_pwconv_workspace_bytes(ctypes.byref(good)) == 2048 + 2 * 32 * 96 * 4
    # the coefficient stride covers both tilings of 300 channels (three tiles of 128 columns, two of 160)
    # and depends on c_out alone: a workspace prepared once serves every batch size and either tiling
    wide = P(dtype=dwlib.F32, c_in=8, c_out=300, h=2, w=2, n=1)
    assert lib.dwbnq_pwconv_workspace_bytes(ctypes.byref(wide)) == 5 * 384 * 4 + 2 * ((8 * 300 * 4 + 255) // 256 * 256)
    deep = P(dtype=dwlib.F32, c_in=512, c_out=300, h=2, w=2, n=1)
    assert lib.dwbnq_pwconv_workspace_bytes(ctypes.byref(deep)) == 5 * 384 * 4 + 2 * 512 * 300 * 4
    for n in (1, 7, 256, 100000):
        again = P(dtype=dwlib.F32, c_in=512, c_out=300, h=14, w=14, n=n)
        assert lib.dwbnq_pwconv_workspace_bytes(ctypes.byref(again)) == 5 * 384 * 4 + 2 * 512 * 300 * 4
    fake, path = ctypes.c_void_p(4096), ctypes.c_int(-1)
    assert lib.dwbnq_pwconv_plan(ctypes.byref(good), fake, fake, ctypes.byref(path)) == dwlib.OK and path.value == 1
    half = P(dtype=dwlib.F16, c_in=32, c_out=96, h=14, w=14, n=4)  # fp16 tensors: gathered, one exact TF32 pass
    assert lib.dwbnq_pwconv_plan(ctypes.byref(half), fake, fake, ctypes.byref(path)) == dwlib.OK and path.value == 1
    for bad in (P(dtype=dwlib.F16, c_in=30, c_out=96, h=14, w=14, n=4),
                P(dtype=dwlib.F32, c_in=30, c_out=96, h=14, w=14, n=4)):  # weight rows not 16-byte multiples
        assert lib.dwbnq_pwconv_plan(ctypes.byref(bad), fake, fake, ctypes.byref(path)) == dwlib.OK and path.value == 0
    # a 7x7 plane is gathered, an unaligned x too: still the tensor-core kernel
    odd = P(dtype=dwlib.F32, c_in=32, c_out=96, h=7, w=7, n=4)
    assert lib.dwbnq_pwconv_plan(ctypes.byref(odd), ctypes.c_void_p(4100), fake, ctypes.byref(path)) == dwlib.OK
    assert path.value == 1
    for kw in ({"dtype": 3}, {"c_in": 0}, {"c_out": -1}, {"h": 0}, {"n": -1}, {"math": 2}, {"act": 3}):
        args = dict(dtype=dwlib.F32, c_in=32, c_out=96, h=14, w=14, n=4)
        args.update(kw)
        d = P(**args)
        assert lib.dwbnq_pwconv_workspace_bytes(ctypes.byref(d)) == 0
        assert lib.dwbnq_pwconv_fwd(ctypes.byref(d), fake, fake, None, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
        assert lib.dwbnq_last_error_string()
    assert lib.dwbnq_pwconv_fwd(None, fake, fake, None, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_pwconv_fwd(ctypes.byref(good), fake, fake, None, fake, fake, -1, None) == dwlib.ERR_INVALID_ARG  # act
    assert lib.dwbnq_set_forced_pw_path(2) == dwlib.ERR_INVALID_ARG
    assert lib.dwbnq_set_pw_max_ctas(-1) == dwlib.ERR_INVALID_ARG
    if lib.dwbnq_device_count() == 0:  # no CPU fallback
        ok = P(dtype=dwlib.F32, c_in=32, c_out=96, h=14, w=14, n=4)
        assert lib.dwbnq_pwconv_fwd(ctypes.byref(ok), fake, fake, None, fake, fake, -1, None) == dwlib.ERR_CUDA


def test_pointwise_launch_shapes_of_the_mobilenet_layers(dwlib):
    """The host-side choices behind a pointwise launch, read back through the debug entry (no device):
    activation path, channel-tile width by the duration estimate, shared-column epilogue."""
    from dwbnq import ops, workloads
    P = dwlib.PwConvDesc
    shape = {}
    for sp in workloads.pw1(256):
        d = P(dtype=dwlib.F32, c_in=sp.c_in, c_out=sp.c_out, h=sp.h, w=sp.h, n=256, math=dwlib.PW_MATH_FP32, act=dwlib.ACT_NONE)
        shape[(sp.c_in, sp.c_out, sp.h)] = ops.pwconv_tiling(d)
    TMA, ONE, FOUR = 0, 1, 2
    for (ci, co, h), s in shape.items():
        assert s["x_path"] == (TMA if h in (112, 56) else ONE if h == 7 else FOUR), (ci, co, h, s)
        assert s["columns"] % 32 == 0 and s["columns"] * s["channel_tiles"] >= co and 2 <= s["stages"] <= 8
        assert s["ctas"] == min(148, s["tiles"]) and s["accumulators"] * s["columns"] <= 512
    # tile widths the estimate picks at this batch (measured: 1.26x, 1.21x, 0.95x - kept narrow - for the three)
    assert shape[(160, 960, 7)]["columns"] == 256 and shape[(160, 960, 7)]["shared_columns"] == 1
    assert shape[(96, 576, 14)]["columns"] == 192 and shape[(96, 576, 14)]["shared_columns"] == 1
    assert shape[(64, 384, 14)]["columns"] == 128 and shape[(64, 384, 14)]["shared_columns"] == 0
    assert shape[(960, 160, 7)]["columns"] == 160 and shape[(960, 160, 7)]["tiles"] == 98
    assert shape[(960, 160, 7)]["shared_columns"] == 1           # one tile per CTA
    assert shape[(16, 96, 112)]["shared_columns"] == 0 and shape[(16, 96, 112)]["accumulators"] == 4
    assert shape[(384, 64, 14)]["shared_columns"] == 1 and shape[(384, 64, 14)]["tiles"] == 392
    # the same layer at two images: narrow tiles again (eight of 128 columns), whatever was prepared
    small = P(dtype=dwlib.F32, c_in=160, c_out=960, h=7, w=7, n=2, math=dwlib.PW_MATH_FP32)
    assert ops.pwconv_tiling(small)["columns"] == 128
    # fp16 tensors: TMA (and binary16 MMAs) where rows are multiples of 16 bytes, else gathered - four positions per
    # load on planes that are multiples of 4 (14 x 14), one element on the others or behind an unaligned x
    half = P(dtype=dwlib.F16, c_in=32, c_out=96, h=56, w=56, n=8)
    assert ops.pwconv_tiling(half)["x_path"] == TMA and ops.pwconv_tiling(half, x_address=4100)["x_path"] == ONE
    assert ops.pwconv_tiling(half, x_address=4104)["x_path"] == FOUR
    assert ops.pwconv_tiling(P(dtype=dwlib.F16, c_in=32, c_out=96, h=28, w=28, n=8))["x_path"] == TMA
    assert ops.pwconv_tiling(P(dtype=dwlib.F16, c_in=64, c_out=96, h=14, w=14, n=8))["x_path"] == FOUR
    assert ops.pwconv_tiling(P(dtype=dwlib.F16, c_in=160, c_out=96, h=7, w=7, n=8))["x_path"] == ONE
    assert ops.pwconv_tiling(P(dtype=dwlib.F16, c_in=20, c_out=96, h=56, w=56, n=8))["x_path"] == FOUR  # w rows of 40 bytes
    odd = P(dtype=dwlib.F32, c_in=32, c_out=96, h=56, w=56, n=8)
    assert ops.pwconv_tiling(odd)["x_path"] == TMA and ops.pwconv_tiling(odd, x_address=4100)["x_path"] == ONE
    # a descriptor for the FMA kernel has no tiling
    with pytest.raises(dwlib.DwbnqError):
        ops.pwconv_tiling(P(dtype=dwlib.F32, c_in=30, c_out=96, h=14, w=14, n=4))
