"""Lane-level CPU emulation of one 16-token step of the CUDA decode kernel (horizon_kernels_b200/csrc/hkv_decode.cu):
the documented register layout of mma.m16n8k16, the kernel's choice of which cache bytes every lane dequantises, the
token permutation of the score tiles and the nibble re-pairing of the value tile. The emulated scores and outputs must
equal a direct dequantise-and-multiply of the same bytes, and two deliberately wrong mappings must fail.
(The reference pins its own kernel the same way: scripts/kernels/kvfp4/test_kvfp4_v2_cpu.py V4 in the reference tree.)
"""
import numpy as np
import pytest

import synth
from oracle import kvfp4 as O


def mma_m16n8k16(a_regs, b_regs, c_regs):
    """a_regs (32, 4, 2), b_regs (32, 2, 2), c_regs (32, 4): registers of f16 pairs per lane -> new c_regs"""
    A = np.zeros((16, 16))
    Bm = np.zeros((16, 8))
    for lane in range(32):
        g, c = lane >> 2, lane & 3
        for i in range(4):
            row = g + 8 * (i & 1)
            col = 2 * c + 8 * (i >> 1)
            A[row, col], A[row, col + 1] = a_regs[lane, i]
        for i in range(2):
            k = 2 * c + 8 * i
            Bm[k, g], Bm[k + 1, g] = b_regs[lane, i]
    Cm = A @ Bm
    out = c_regs.copy()
    for lane in range(32):
        g, c = lane >> 2, lane & 3
        out[lane, 0] += Cm[g, 2 * c]
        out[lane, 1] += Cm[g, 2 * c + 1]
        out[lane, 2] += Cm[g + 8, 2 * c]
        out[lane, 3] += Cm[g + 8, 2 * c + 1]
    return out


E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])


def cvt_byte(b):
    """cvt.rn.f16x2.e2m1x2: low nibble -> low half"""
    return E2M1[b & 15], E2M1[b >> 4]


class Geo:
    def __init__(self, D, layout):
        self.D, self.layout = D, layout
        self.SD, self.SS = D // 2, D // 16
        self.SLOT = self.SD + self.SS
        self.ROW = self.SLOT if layout == 0 else self.SD
        self.SF_BASE = self.SD if layout == 0 else 16 * self.SD
        self.SF_ROW = self.SLOT if layout == 0 else self.SS
        self.KS, self.NBL, self.NH = D // 16, D // 64, D // 128

    def tok(self, i):
        if self.D == 128 and self.layout == 0:
            return (i & 5) | ((i & 2) << 2) | ((i & 8) >> 2)       # bits 1 and 3 swapped
        return i

    def kblk(self, c, u):
        return self.NBL * c + u


def movmatrix_trans(regs):
    """movmatrix.sync.aligned.m8n8.trans.b16: lane l holds row l // 4, columns 2 (l % 4), 2 (l % 4) + 1"""
    m = np.zeros((8, 8))
    for lane in range(32):
        m[lane >> 2, 2 * (lane & 3)], m[lane >> 2, 2 * (lane & 3) + 1] = regs[lane]
    out = np.zeros_like(regs)
    for lane in range(32):
        out[lane] = m.T[lane >> 2, 2 * (lane & 3)], m.T[lane >> 2, 2 * (lane & 3) + 1]
    return out


def make_tile(seed, geo):
    """one (head, side) tile of 16 tokens in the kernel's shared-memory byte order, plus its dequantised matrix"""
    x = (synth.normal(seed, (16, geo.D)) * 3).astype(np.float32)
    data, sf = O.quantize_rows(x, 1.0)
    deq = O.dequantize_rows(data, sf)
    tile = np.zeros(16 * geo.SLOT, np.uint8)
    for r in range(16):
        tile[r * geo.ROW:r * geo.ROW + geo.SD] = data[r]
        tile[geo.SF_BASE + r * geo.SF_ROW:geo.SF_BASE + r * geo.SF_ROW + geo.SS] = sf[r]
    return tile, deq


def emulate_unit(geo, kt, vt, q, wrong=None):
    """q (8, D) float. Returns S (8 rows, 16 tokens) and O (8 rows, D) accumulated with P = S (no softmax), exactly as
    the kernel's fragments would hold them."""
    D = geo.D
    sf_val = O.e4m3_decode(np.arange(256, dtype=np.uint8))
    # query fragments qa[lane][kstep][2 regs][2 halves]: row g, channels of the lane's key blocks
    qa = np.zeros((32, geo.KS, 2, 2))
    for lane in range(32):
        g, c = lane >> 2, lane & 3
        for u in range(geo.NBL):
            ch0 = 16 * geo.kblk(c, u)
            for i in range(8):
                qa[lane, 4 * u + (i >> 1), i & 1] = q[g, ch0 + 2 * i], q[g, ch0 + 2 * i + 1]
    st = np.zeros((32, 4))                             # S^T tile: rows = tokens, columns = query rows
    for u in range(geo.NBL):
        e = np.zeros((2, 32, 8, 2))                  # [token of the lane][lane][byte of the block][half]
        for lane in range(32):
            g, c = lane >> 2, lane & 3
            kb = geo.kblk(c, u)
            if wrong == "kblock" and u == 0:
                kb = geo.kblk((c + 1) % 4, u)
            for t in range(2):
                r = geo.tok(g + 8 * t)
                scale = sf_val[kt[geo.SF_BASE + r * geo.SF_ROW + kb]]
                for by in range(8):
                    lo, hi = cvt_byte(int(kt[r * geo.ROW + 8 * kb + by]))
                    e[t, lane, by] = lo * scale, hi * scale
        for v in range(4):
            a = np.stack([e[0, :, 2 * v], e[1, :, 2 * v], e[0, :, 2 * v + 1], e[1, :, 2 * v + 1]], axis=1)
            st = mma_m16n8k16(a, qa[:, 4 * u + v], st)
    S = np.zeros((8, 16))
    for lane in range(32):
        g, c = lane >> 2, lane & 3
        S[2 * c, geo.tok(g)], S[2 * c + 1, geo.tok(g)] = st[lane, 0], st[lane, 1]
        S[2 * c, geo.tok(g + 8)], S[2 * c + 1, geo.tok(g + 8)] = st[lane, 2], st[lane, 3]
    pb = np.stack([movmatrix_trans(st[:, 0:2]), movmatrix_trans(st[:, 2:4])], axis=1)
    o = np.zeros((geo.KS, 32, 4))
    for hf in range(geo.NH):
        for jj in range(8):
            a = np.zeros((32, 4, 2))
            for lane in range(32):
                g, c = lane >> 2, lane & 3
                vb = g + 8 * hf
                toks = [geo.tok(2 * c), geo.tok(2 * c + 1), geo.tok(2 * c + 8), geo.tok(2 * c + 9)]
                if wrong == "vtokens":
                    toks[0], toks[1] = toks[1], toks[0]
                w = [vt[t * geo.ROW + 8 * vb:t * geo.ROW + 8 * vb + 8].astype(np.int64) for t in toks]
                f = [sf_val[vt[geo.SF_BASE + t * geo.SF_ROW + vb]] for t in toks]
                for pair in range(2):
                    w0, w1 = w[2 * pair], w[2 * pair + 1]
                    xe = (w0 & 15) | ((w1 & 15) << 4)         # even channels: low nibble = first token of the pair
                    xo = (w0 >> 4) | (w1 & 0xF0)              # odd channels
                    lo, hi = cvt_byte(int(xe[jj]))
                    a[lane, 2 * pair] = lo * f[2 * pair], hi * f[2 * pair + 1]
                    lo, hi = cvt_byte(int(xo[jj]))
                    a[lane, 2 * pair + 1] = lo * f[2 * pair], hi * f[2 * pair + 1]
            o[8 * hf + jj] = mma_m16n8k16(a, pb, o[8 * hf + jj])
    Om = np.zeros((8, D))
    for lane in range(32):
        g, c = lane >> 2, lane & 3
        for hf in range(geo.NH):
            for jj in range(8):
                ch = 16 * (g + 8 * hf) + 2 * jj
                a = o[8 * hf + jj][lane]
                Om[2 * c, ch], Om[2 * c, ch + 1] = a[0], a[2]
                Om[2 * c + 1, ch], Om[2 * c + 1, ch + 1] = a[1], a[3]
    return S, Om


@pytest.mark.parametrize("D,layout", [(128, 0), (128, 1), (256, 0), (256, 1)])
def test_unit_mapping(D, layout):
    geo = Geo(D, layout)
    kt, kdeq = make_tile(10 + D + layout, geo)
    vt, vdeq = make_tile(20 + D + layout, geo)
    q = synth.bf16_bits_to_f32(synth.to_bf16_bits(synth.normal(30 + D, (8, D)))).astype(np.float64)
    S, Om = emulate_unit(geo, kt, vt, q)
    S_ref = q @ kdeq.T
    assert np.abs(S - S_ref).max() <= 1e-9 * np.abs(S_ref).max()
    O_ref = S_ref @ vdeq
    assert np.abs(Om - O_ref).max() <= 1e-9 * np.abs(O_ref).max()


@pytest.mark.parametrize("wrong", ["kblock", "vtokens"])
def test_negative_controls(wrong):
    geo = Geo(128, 0)
    kt, kdeq = make_tile(41, geo)
    vt, vdeq = make_tile(42, geo)
    q = synth.normal(43, (8, 128))
    S, Om = emulate_unit(geo, kt, vt, q, wrong=wrong)
    S_ref = q @ kdeq.T
    O_ref = S_ref @ vdeq
    err = max(np.abs(S - S_ref).max() / np.abs(S_ref).max(), np.abs(Om - O_ref).max() / np.abs(O_ref).max())
    assert err > 0.05


def _wavefronts(addrs, width):
    """shared-memory passes of one warp-wide load: 4-byte banks, a pass serves every lane whose words do not collide;
    8-byte loads are served per half warp and 16-byte loads per quarter warp"""
    group = {1: 32, 2: 32, 4: 32, 8: 16, 16: 8}[width]
    total = 0
    for s0 in range(0, 32, group):
        words = {}
        for a in addrs[s0:s0 + group]:
            for wd in range(a // 4, (a + width + 3) // 4):
                words.setdefault(wd % 32, set()).add(wd)
        total += max(len(v) for v in words.values())
    return total


@pytest.mark.parametrize("D", [128, 256])
def test_shared_memory_loads_are_conflict_free(D):
    """every load pattern of the slot layout (key codes and scales, value codes and scales) takes the minimum number
    of shared-memory passes"""
    geo = Geo(D, 0)
    lanes = [(lane >> 2, lane & 3) for lane in range(32)]
    for row in (0, 8):
        if D == 128:
            for u in range(2):
                assert _wavefronts([geo.tok(g + row) * geo.ROW + 8 * geo.kblk(c, u) for g, c in lanes], 8) == 2
            assert _wavefronts([geo.SF_BASE + geo.tok(g + row) * geo.SF_ROW + geo.kblk(c, 0) for g, c in lanes], 2) == 1
        else:
            for j in range(2):
                assert _wavefronts([geo.tok(g + row) * geo.ROW + 8 * geo.kblk(c, 0) + 16 * j for g, c in lanes], 16) == 4
            assert _wavefronts([geo.SF_BASE + geo.tok(g + row) * geo.SF_ROW + geo.kblk(c, 0) for g, c in lanes], 4) == 1
    for hf in range(geo.NH):
        for off in (0, 1, 8, 9):
            assert _wavefronts([geo.tok(2 * c + off) * geo.ROW + 8 * g + 64 * hf for g, c in lanes], 8) == 2
            assert _wavefronts([geo.SF_BASE + geo.tok(2 * c + off) * geo.SF_ROW + g + 8 * hf for g, c in lanes], 1) == 1


def test_row_offsets_are_lane_independent():
    """the kernel addresses a lane's second key row and its other three value rows by constants"""
    for D in (128, 256):
        for layout in (0, 1):
            geo = Geo(D, layout)
            assert len({geo.tok(g + 8) - geo.tok(g) for g in range(8)}) == 1
            for off in (1, 8, 9):
                assert len({geo.tok(2 * c + off) - geo.tok(2 * c) for c in range(4)}) == 1
            assert sorted(geo.tok(i) for i in range(16)) == list(range(16))
