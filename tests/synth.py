"""Deterministic synthetic inputs for the parity tests: a counter-based generator (splitmix64 -> Box-Muller) written
in numpy, so the same seed gives the same bf16 tensors on every machine, with no dependence on a library's RNG stream.
The golden fixtures under tests/golden/ were produced from these inputs."""
import math

import numpy as np

_M = (1 << 64) - 1


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int) -> np.ndarray:
    """n float64 in (0, 1)"""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64) + np.uint64((seed * 0x1000003D + 0x51ED270B) & _M)
        z = _splitmix64(_splitmix64(idx))
    return ((z >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def normal(seed: int, shape) -> np.ndarray:
    """float64 standard normal of the given shape"""
    n = int(np.prod(shape))
    m = (n + 1) // 2
    u1, u2 = uniform(2 * seed + 1, m), uniform(2 * seed + 2, m)
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.concatenate([r * np.cos(2 * math.pi * u2), r * np.sin(2 * math.pi * u2)])[:n]
    return out.reshape(shape)


def permutation(seed: int, n: int) -> np.ndarray:
    return np.argsort(uniform(seed, n), kind="stable").astype(np.int64)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float -> bf16 bit patterns (uint16), round to nearest even"""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def paged_case(seed, lens, KVH, G, D, PS, QL=1, outliers=False, extra_pages=3, ql_list=None):
    """A decode case in the style of the reference's GPU tests (test_kvfp4_gpu.py:81-110 in the reference): a page
    table drawn from a permutation that never uses page 0, keys optionally with 4 outlier channels per head scaled by
    20, bf16 q / k / v. Returns a dict of numpy arrays (bf16 as uint16 bit patterns)."""
    B = len(lens)
    pages = [math.ceil(L / PS) for L in lens]
    NP = sum(pages) + extra_pages
    perm = permutation(seed * 7 + 1, NP - 1) + 1
    MP = max(1, max(pages) if pages else 1)
    bt = np.zeros((B, MP), np.int32)
    o = 0
    for b, p in enumerate(pages):
        bt[b, :p] = perm[o:o + p]
        o += p
    slots = np.array([int(bt[b, p // PS]) * PS + p % PS for b, L in enumerate(lens) for p in range(L)], np.int64)
    NT = int(sum(lens))
    k = normal(seed * 7 + 2, (NT, KVH, D))
    v = normal(seed * 7 + 3, (NT, KVH, D))
    if outliers:
        ch = (np.arange(4) * (D // 4) + 3) % D
        k[:, :, ch] *= 20.0
    qls = list(ql_list) if ql_list is not None else [QL] * B
    qsl = np.zeros(B + 1, np.int32)
    qsl[1:] = np.cumsum(qls)
    q = normal(seed * 7 + 4, (int(qsl[-1]), KVH * G, D))
    return dict(NP=NP, bt=bt, slots=slots, key=to_bf16_bits(k), val=to_bf16_bits(v), q=to_bf16_bits(q),
                seq_lens=np.array(lens, np.int32), qsl=qsl, KVH=KVH, G=G, D=D, PS=PS)


def tensor_scale(bits: np.ndarray) -> float:
    """fp32 per-tensor global scale amax / (6 * 448) of a bf16 tensor given as bit patterns"""
    amax = np.float32(np.abs(bf16_bits_to_f32(bits)).max()) if bits.size else np.float32(1.0)
    return float(np.float32(amax) / np.float32(6.0 * 448.0))
