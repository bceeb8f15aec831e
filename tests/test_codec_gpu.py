"""Exhaustive checks of the hardware conversions the kernels stand on, run on the GPU through the C ABI
(hkv_selftest_codec). The reference pins the equivalent bit formulas of its own kernels exhaustively on the CPU
(scripts/kernels/kvfp4/test_kvfp4_cpu.py:54-99 and :390-434, test_kvfp4_serving_cpu.py:47-110 in the reference); here
the formulas are machine instructions, so the check has to run where they execute.

  * write side: cvt.rn.satfinite.e2m1x2.f32 against the reference's threshold chain (kv_fp4_ref.py:122-130) for EVERY
    non-negative fp32 bit pattern from 0 to +inf; the quotient by three multiply-adds with the scale's reciprocal
    against the IEEE division the reference performs, over 6 * 10^7 (value, scale) pairs;
  * read side: cvt.rn.f16x2.e2m1x2(code) * cvt.rn.f16x2.e4m3x2(scale byte) in f16 against e2m1_value * e4m3_value for
    all 16 codes x 256 scale bytes (the product is exact in f16); 0x7f / 0xff are NaN in E4M3 and stay NaN."""
import ctypes as C

import numpy as np
import pytest
import torch

from horizon_kernels_b200 import _lib

pytestmark = pytest.mark.gpu

NBYTES = 64 + 16 * 256 * 2


@pytest.fixture(scope="module")
def selftest():
    buf = torch.full((NBYTES,), 0xEE, dtype=torch.uint8, device="cuda")
    rc = _lib.load().hkv_selftest_codec(C.c_void_p(buf.data_ptr()), NBYTES,
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    host = buf.cpu().numpy()
    return host[:64].view(np.uint64), host[64:].view(np.uint16).reshape(16, 256)


def test_hardware_e2m1_encode_equals_the_threshold_chain_for_every_non_negative_float(selftest):
    counts, _ = selftest
    assert int(counts[0]) == 0          # 0 .. +inf: 2^31 - 2^23 + 1 bit patterns, none differs
    # NaN inputs: the threshold chain saturates them to code 7 (every comparison is false) and so does the hardware
    assert int(counts[1]) == 0


def test_quotient_by_multiply_adds_equals_the_division(selftest):
    """the write kernel never divides a value by its scale: y0 = a * r, rem = fma(-s, y0, a), q = fma(rem, r, y0) with
    r = RN(1 / s); the result must be the IEEE quotient the reference computes (kv_fp4_ref.py:159-186)"""
    counts, _ = selftest
    assert int(counts[3]) > 5 * 10 ** 7          # the pairs that were inside the fast path's range and compared
    assert int(counts[2]) == 0


def test_packed_pair_error_sum_equals_the_chain_of_single_operations(selftest):
    """codes and squared error of a block from the packed fp32 pair instructions (mul.f32x2 / fma.f32x2) against the
    reference's order of single IEEE operations (kv_fp4_ref.py:148-156): bit-equal, so the scale search picks the same
    candidate even where two errors differ by one ulp (an assembler that contracts a packed multiply with the packed
    subtraction after it rounds once instead of twice and fails this)"""
    counts, _ = selftest
    assert int(counts[5]) > 10 ** 6
    assert int(counts[4]) == 0


def test_dequantised_product_table_is_exact(selftest):
    _, table = selftest
    got = table.view(np.float16).astype(np.float64)
    e2m1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float64)
    code_val = np.concatenate([e2m1, -e2m1])                              # bit 3 is the sign
    b = np.arange(256)
    e, m = (b >> 3) & 15, b & 7
    mag = np.where(e > 0, (1 + m / 8.0) * 2.0 ** (e - 7), m * 2.0 ** -9)  # e4m3fn: bias 7, subnormals m * 2^-9
    sc = np.where(b & 0x80, -mag, mag)
    want = code_val[:, None] * sc[None, :]
    nan_cols = (b & 0x7F) == 0x7F                                         # 0x7f and 0xff are NaN, there is no infinity
    assert np.isnan(got[:, nan_cols]).all()
    ok = ~nan_cols
    assert np.array_equal(got[:, ok], want[:, ok])
    # signed zeros: a zero code or a zero scale gives a zero of either sign, never anything else
    assert (got[0, ok] == 0).all() and (got[:, 0] == 0).all()
    # the largest product a written cache can hold: code 6 * scale 448
    assert got[7, 0x7E] == 2688.0


def test_selftest_rejects_misuse():
    L = _lib.load()
    buf = torch.zeros(NBYTES, dtype=torch.uint8, device="cuda")
    assert L.hkv_selftest_codec(None, NBYTES, None) == -1
    assert L.hkv_selftest_codec(C.c_void_p(buf.data_ptr()), NBYTES - 1, None) == -5
    assert L.hkv_selftest_codec(C.c_void_p(buf.data_ptr() + 4), NBYTES, None) == -2


def test_issue_rate_probe_runs_and_orders_the_pipes():
    """the probe behind the decode kernel's design notes: fp32 fma issues at full rate, the E2M1 conversion and the f16x2
    multiply at about half of it, and the dequantise group costs more with its warp-level mma than without"""
    L = _lib.load()
    M = 12
    nbytes = M * 256 * 8 + 256 * 1024 * 4
    buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    assert L.hkv_probe_issue_rates(C.c_void_p(buf.data_ptr()), nbytes, 4, None) == 0
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    cyc = buf[:M * 256 * 8].view(torch.int64).view(M, 256)[:, :sms].double().mean(dim=1).cpu().numpy()
    per = cyc / (2048 * np.array([8, 8, 8, 8, 8, 9, 10, 8, 8, 8, 8, 8]) * 4)
    assert (per > 0.2).all() and (per < 20).all()
    assert per[2] < per[0] and per[2] < per[1]                 # fma.f32 is faster than the conversion and the f16x2 multiply
    assert cyc[6] > cyc[5]                                     # the mma adds issue time to the group
    assert 1.5 * per[7] < per[8] < 2.5 * per[7]                # a packed mul.f32x2 holds the pipe like two fp32 multiplies
    assert L.hkv_probe_issue_rates(C.c_void_p(buf.data_ptr()), nbytes, 9, None) == -6
    assert L.hkv_probe_issue_rates(C.c_void_p(buf.data_ptr()), 16, 4, None) == -5
