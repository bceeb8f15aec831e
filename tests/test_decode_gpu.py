"""GPU parity of the split-K decode + combine kernels, through the C ABI, against the reference's fp64 attention over
the same dequantised cache (golden fixtures) and against the CPU oracle. Tolerances are the task's: max-abs 2e-2,
mean-abs 2e-3, and the reference's own gate, relative L2 2.5e-3 (scripts/kernels/kvfp4/test_kvfp4_gpu.py:51).
Mirrors the reference's decode gates G3 / G3v2 / S1: partial pages, garbage bytes (0x7F = NaN as E4M3) outside the
written slots, non-unit global scales, a padded output buffer, determinism, NaN-poisoned CUDA-graph replay."""
import os

import numpy as np
import pytest
import torch

import synth
from cases import (Cache, assert_close, bf16_tensor, build_decode_case, errors, gpu_decode, oracle_decode,
                   unquantised_attention)
from horizon_kernels_b200 import kernels as K
from horizon_kernels_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["g4", "g8"])
def test_attention_golden(golden_dir, name):
    """the reference's own attention_reference output on a cache the reference wrote"""
    z = np.load(os.path.join(golden_dir, "attention.npz"))
    KVH, G, D, PS, QL, NP = (int(v) for v in z[f"{name}_geom"])
    cache = Cache(NP, PS, KVH, D, "region")
    cache.load(z[f"{name}_cache"])
    sm, vs = (float(v) for v in z[f"{name}_sm"])
    c = dict(cache=cache, q=z[f"{name}_q"], bt=z[f"{name}_bt"], seq_lens=z[f"{name}_seq_lens"], qsl=z[f"{name}_qsl"],
             gk=z[f"{name}_gk"], gv=z[f"{name}_gv"], KVH=KVH, G=G, D=D, sm=sm)
    out, ws = gpu_decode(c, v_scale=vs)
    assert K.workspace_status(ws) == 0
    assert_close(out, z[f"{name}_ref"], name)


def test_config0_golden(golden_dir):
    """batch 4, 32 / 8 heads, head_dim 128, 2048 tokens each, 512 pages: cache bytes equal to the reference's
    (sha256) and attention within tolerance of the reference's fp64 output"""
    import hashlib
    from test_oracle import config0_inputs
    z = np.load(os.path.join(golden_dir, "config0.npz"))
    c = config0_inputs()
    cache = Cache(512, 16, 8, 128, "region", fill=0)
    dev = cache.phys.device
    K.write(bf16_tensor(c["key"]), bf16_tensor(c["val"]), cache.flat, cache.strides, 16,
            torch.from_numpy(c["slots"]).to(dev), torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev))
    assert hashlib.sha256(cache.bytes().tobytes()).hexdigest() == str(z["cache_sha256"])
    c.update(cache=cache, sm=float(z["sm"][0]))
    out, ws = gpu_decode(c)
    assert K.workspace_status(ws) == 0
    mx, mn, rl = assert_close(out, z["ref"], "config0")
    print("config0 errors", mx, mn, rl)


CASES = [
    # lens, KVH, G, D, PS, layout
    ([37], 8, 4, 128, 16, "hnd"),
    ([1, 5, 17, 16, 15, 33], 8, 4, 128, 16, "hnd"),
    ([1601, 7, 900], 8, 4, 128, 16, "hnd"),
    ([300, 1000], 8, 8, 128, 16, "hnd"),
    ([5, 64, 200, 0, 129], 2, 8, 256, 16, "hnd"),
    ([20000, 7], 2, 8, 256, 16, "hnd"),
    ([129, 300], 4, 6, 256, 64, "hnd"),
    ([129, 300, 70], 4, 6, 256, 64, "region"),
    ([150, 16, 2048], 8, 4, 128, 16, "region"),
    ([500, 40], 3, 5, 128, 32, "hnd"),
    ([700], 1, 1, 128, 16, "hnd"),
]


@pytest.mark.parametrize("lens,KVH,G,D,PS,kind", CASES)
def test_decode_matches_oracle(lens, KVH, G, D, PS, kind):
    c = build_decode_case(1000 + len(lens) + KVH + G, lens, KVH, G, D, PS, kind=kind, gscale=(0.05, 0.01))
    ref = oracle_decode(c, v_scale=0.5)
    NT = c["q"].shape[0]
    out = torch.full((NT + 3, KVH * G, D), 7.0, dtype=torch.bfloat16, device="cuda")      # padded output buffer
    out, ws = gpu_decode(c, v_scale=0.5, out=out)
    assert K.workspace_status(ws) == 0
    assert_close(out, ref, str(lens))
    assert (out[NT:] == 7.0).all()                               # rows past the query tokens are untouched
    out2 = torch.full_like(out, 7.0)
    gpu_decode(c, v_scale=0.5, out=out2, ws=ws)
    assert torch.equal(out, out2)                                # deterministic
    for splits in (1, 2, 64):
        o3 = torch.full_like(out, 7.0)
        gpu_decode(c, v_scale=0.5, out=o3, ws=ws, splits=splits)
        assert_close(o3, ref, f"{lens} splits {splits}")


def test_large_ragged_batch():
    """300 requests, lengths log-uniform in [1, 3000] with some empty contexts and some padding requests (0 query
    tokens): the per-CTA prefix scan spans several 32-request groups and most partitions hold many short sequences"""
    B = 300
    u = synth.uniform(555, B)
    lens = [int(np.exp(x * np.log(3000.0))) for x in u]
    for i in range(0, B, 37):
        lens[i] = 0
    qls = [0 if i % 41 == 5 else 1 for i in range(B)]
    for D, KVH, G in ((128, 8, 4), (256, 2, 8)):
        c = build_decode_case(2500 + D, lens, KVH, G, D, 16, ql_list=qls)
        ref = oracle_decode(c)
        out, ws = gpu_decode(c)
        assert K.workspace_status(ws) == 0
        assert_close(out, ref, f"D{D}")
        out2, _ = gpu_decode(c, ws=ws)
        assert torch.equal(out, out2)


def test_rows_without_query_tokens_are_untouched():
    """a graph-padding request (0 query tokens) and a prefill row (more than qlmax tokens) are skipped"""
    lens = [40, 300, 64, 90]
    c = build_decode_case(2000, lens, 8, 4, 128, 16, ql_list=[1, 0, 1, 3])
    ref = oracle_decode(c)
    NT = c["q"].shape[0]
    out = torch.full((NT, 32, 128), 3.0, dtype=torch.bfloat16, device="cuda")
    out, _ = gpu_decode(c, out=out, qlmax=1)
    q0 = c["qsl"]
    prefill_rows = slice(int(q0[3]), int(q0[4]))
    assert (out[prefill_rows] == 3.0).all()
    ref[prefill_rows] = np.nan
    assert_close(out, ref)


def test_two_query_tokens_causal():
    """MTP-style rows: 2 query tokens with 4 heads per kv head fit the 8-row tile; token t sees L - 2 + t + 1 keys"""
    c = build_decode_case(2100, [50, 333, 17], 8, 4, 128, 16, ql_list=[2, 2, 1])
    ref = oracle_decode(c)
    out, _ = gpu_decode(c, qlmax=2)
    assert_close(out, ref)


def test_early_metadata_option_changes_nothing():
    """with HKV_OPT_EARLY_METADATA the kernel reads seq_lens / query_start_loc ahead of its launch dependency; when they
    are old enough (here: written long before, a synchronize in between) the output is bit-identical, also when decode
    launches follow one another back to back"""
    lens = [777, 16, 4100, 0, 95, 2048]
    c = build_decode_case(2300, lens, 8, 4, 128, 16)
    ref = oracle_decode(c)
    K.set_option(K.OPT_EARLY_METADATA, 0)
    out0, ws = gpu_decode(c)
    torch.cuda.synchronize()
    try:
        K.set_option(K.OPT_EARLY_METADATA, 1)
        outs = []
        for _ in range(4):                                       # back to back: launch k + 1 overlaps the tail of launch k
            o = torch.zeros_like(out0)
            gpu_decode(c, out=o, ws=ws)
            outs.append(o)
        torch.cuda.synchronize()
        assert K.workspace_status(ws) == 0
        for o in outs:
            assert torch.equal(o, out0)
    finally:
        K.set_option(K.OPT_EARLY_METADATA, 0)
    assert_close(out0, ref)


def test_error_against_unquantised_fp64_attention():
    """the "float64 oracle" column: error of the whole 4-bit path (quantise, decode) against fp64 attention over the
    unquantised bf16 K / V, config-0 shape (batch 4, 32 / 8 heads, head_dim 128, 2048 tokens, N(0,1) data, global scale
    amax / (6 * 448)). The GPU result must not add error beyond the format's: it stays as close to the unquantised
    truth as the reference's own fp64 attention over the same cache does."""
    c = build_decode_case(2350, [2048] * 4, 8, 4, 128, 16, outliers=False)
    out, _ = gpu_decode(c)
    ref = oracle_decode(c)
    true = unquantised_attention(c, c["sm"])
    got = out.float().cpu().numpy().astype(np.float64)
    e_gpu = np.linalg.norm(got - true) / np.linalg.norm(true)
    e_ref = np.linalg.norm(ref - true) / np.linalg.norm(true)
    print("relative L2 vs unquantised fp64 attention: gpu %.4f, fp64 attention over the cache %.4f" % (e_gpu, e_ref))
    assert e_gpu <= e_ref * 1.02 + 1e-3 and e_gpu < 0.2


def test_long_context_split_and_combine():
    """64k tokens on one kv head pair: the sequence is cut over every partition and merged by the CTA that finishes last"""
    c = build_decode_case(2200, [65536], 2, 8, 128, 16)
    ref = oracle_decode(c)
    out, ws = gpu_decode(c)
    assert K.workspace_status(ws) == 0
    mx, mn, rl = assert_close(out, ref)
    print("64k errors", mx, mn, rl)


@pytest.mark.parametrize("D,KVH,G", [(128, 2, 4), (256, 1, 8), (128, 2, 8)])
def test_every_sequence_split_over_three_or_more_partitions(D, KVH, G):
    """few long sequences on a grid that fills the GPU: every sequence is cut into many pieces (hundreds of partitions
    over 2 to 4 sequences), each merged inside the decode launch by whichever CTA finishes its last piece. The result
    must not depend on which CTA that is: three runs are bit-equal, the ticket counters are back at zero after every
    launch, and a cap on the partitions (`splits` 1 / 2 / 64, i.e. 1, 2 and up to 64 pieces per sequence) stays within
    the tolerance."""
    lens = [9000, 12345]
    one_pass = 16 if D == 128 else 8                  # query rows per kv head a single pass serves
    two = G * 2 <= one_pass                            # (group 8 x 2 tokens at head_dim 128: the sixteen-row kernel)
    c = build_decode_case(2210 + D + G, lens, KVH, G, D, 16, ql_list=[1, 2] if two else None)
    ref = oracle_decode(c, v_scale=0.5)
    qlmax = 2 if two else 1
    out, ws = gpu_decode(c, v_scale=0.5, qlmax=qlmax)
    assert K.workspace_status(ws) == 0
    assert_close(out, ref)
    tickets = ws[256:256 + 4 * 2 * K.num_sms()].view(torch.int32)   # the counters of the first 2 * SMs partitions
    assert int(tickets.abs().sum()) == 0
    for _ in range(2):
        o2 = torch.full_like(out, float("nan"))
        gpu_decode(c, v_scale=0.5, out=o2, ws=ws, qlmax=qlmax)
        assert torch.equal(o2, out)
        assert int(tickets.abs().sum()) == 0
    for splits in (1, 2, 64):
        o3 = torch.full_like(out, float("nan"))
        gpu_decode(c, v_scale=0.5, out=o3, ws=ws, splits=splits, qlmax=qlmax)
        assert_close(o3, ref, f"splits {splits}")
        assert int(tickets.abs().sum()) == 0


def test_graph_replay_with_poisoned_output():
    c = build_decode_case(2300, [700, 33, 4000, 16], 8, 4, 128, 16)
    ref = oracle_decode(c)
    out, ws = gpu_decode(c)
    torch.cuda.synchronize()
    first = out.clone()
    assert_close(first, ref)
    dev = out.device
    q = bf16_tensor(c["q"])
    bt, sl, qsl = (torch.from_numpy(c[k]).to(dev) for k in ("bt", "seq_lens", "qsl"))
    gk, gv = torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev)
    cache = c["cache"]

    def run():
        K.decode_ragged(q, cache.flat, cache.strides, cache.PS, bt, sl, qsl, c["sm"], 1.0, gk, gv, 1, out, ws)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        run()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            run()
    for _ in range(2):
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, first)
    # the same graph serves other context lengths: shrink two requests on the device and replay
    sl2 = c["seq_lens"].copy()
    sl2[0], sl2[2] = 123, 1999
    sl.copy_(torch.from_numpy(sl2))
    g.replay()
    torch.cuda.synchronize()
    c2 = dict(c, seq_lens=sl2)
    assert_close(out, oracle_decode(c2))


@pytest.mark.parametrize("KVH,G,D,qls", [(2, 16, 128, [1, 1, 1]), (8, 4, 128, [4, 2, 4]), (2, 8, 256, [3, 1, 2]),
                                         (1, 12, 128, [5, 5, 1])])
def test_more_than_eight_query_rows(KVH, G, D, qls):
    """G * ql > 8 rows per kv head (large groups, several draft tokens): served eight rows per pass over the cache;
    causal among the request's own query tokens; requests with fewer query tokens drop out of the later passes"""
    lens = [333, 40, 1500][:len(qls)]
    c = build_decode_case(2450 + G, lens, KVH, G, D, 16, ql_list=qls)
    ref = oracle_decode(c)
    NT = c["q"].shape[0]
    out = torch.full((NT + 2, KVH * G, D), 5.0, dtype=torch.bfloat16, device="cuda")
    out, ws = gpu_decode(c, out=out, qlmax=max(qls))
    assert K.workspace_status(ws) == 0
    assert_close(out, ref, f"G{G} ql{qls}")
    assert (out[NT:] == 5.0).all()
    out2 = torch.full_like(out, 5.0)
    gpu_decode(c, out=out2, ws=ws, qlmax=max(qls), splits=2)
    assert_close(out2, ref, "splits 2")


def test_length_beyond_the_block_table_is_cut_at_its_reach():
    """seq_lens larger than MP * PS (bad metadata) must not read past the block-table row: the kernel uses MP * PS"""
    c = build_decode_case(2460, [112, 64], 2, 4, 128, 16)
    MP = c["bt"].shape[1]
    full = dict(c, seq_lens=np.array([MP * 16, 64], np.int32), bt=c["bt"].copy())
    if MP * 16 > 112:                                            # pages past the context: point them at page 0 (written)
        full["bt"][0, 7:] = c["bt"][0, 0]
    want, _ = gpu_decode(full)
    bad = dict(full, seq_lens=np.array([1 << 30, 64], np.int32))
    got, ws = gpu_decode(bad)
    assert K.workspace_status(ws) == 0
    assert torch.equal(got, want)


def test_bounded_wait_reports_instead_of_hanging():
    """the failure path of every device-side wait: a wait on a barrier that nothing completes gives up after its limit
    (here 2 million cycles, about a millisecond), records HKV_ERR_DEVICE_WAIT in the workspace header, the kernel ends,
    and the same workspace then serves a normal decode"""
    import ctypes as C
    c = build_decode_case(2470, [100], 2, 4, 128, 16)
    ws = K.alloc_workspace(1, 2, 4, 128, 1, "cuda")
    L = _lib.load()
    rc = L.hkv_selftest_wait_timeout(C.c_void_p(ws.data_ptr()), 2_000_000,
                                     C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    assert K.workspace_status(ws) == -8                          # HKV_ERR_DEVICE_WAIT, cleared by the read
    assert K.workspace_status(ws) == 0
    out, _ = gpu_decode(c, ws=ws)
    assert K.workspace_status(ws) == 0
    assert_close(out, oracle_decode(c))


def test_unsupported_shapes_raise():
    with pytest.raises(_lib.HkvError):
        K.alloc_workspace(1, 1, 65, 128, 1)                                # more than 64 query rows per kv head
    with pytest.raises(_lib.HkvError):
        K.alloc_workspace(1, 1, 4, 96, 1)                                  # head_dim outside {128, 256}


@pytest.mark.parametrize("lens,KVH,G,D,PS", [([40, 1601, 7], 8, 4, 128, 16), ([333, 16, 2048], 3, 4, 128, 32),
                                             ([129, 300, 70, 5000], 2, 8, 256, 16), ([700, 64], 4, 6, 256, 64)])
@pytest.mark.parametrize("writer", ["gpu", "oracle"])
def test_positions_outermost_pages(lens, KVH, G, D, PS, writer):
    """vLLM's other page order (positions outermost inside a page, NHD: the reference advertises both,
    backend.py:107-110, and its kernels take any strides, kv_fp4_serving.py:873-886): a head's token rows are not
    back to back, so the decode copies them row by row. Same numbers as over head-major pages of the same tokens,
    bit for bit, and within tolerance of the oracle; odd kv head counts put the value rows off the 16-byte grid."""
    c = build_decode_case(2600 + D + PS, lens, KVH, G, D, PS, kind="nhd", writer=writer)
    ref = oracle_decode(c, v_scale=0.5)
    out, ws = gpu_decode(c, v_scale=0.5)
    assert K.workspace_status(ws) == 0
    assert_close(out, ref, f"nhd {lens}")
    c2 = build_decode_case(2600 + D + PS, lens, KVH, G, D, PS, kind="hnd", writer=writer)
    out2, _ = gpu_decode(c2, v_scale=0.5)
    assert torch.equal(out, out2)
    o3, _ = gpu_decode(c, v_scale=0.5, ws=ws, splits=2)
    assert_close(o3, ref, "splits 2")


def test_minimal_workspace_of_a_capped_split_count():
    """a C caller that caps the partitions with `splits` may pass the smaller workspace that count needs: 1 request x
    1 kv head x splits 1 = one partition = 25088 bytes at head_dim 128. The call must stay inside it (canary bytes behind
    it untouched), give the right output, and refuse a workspace one byte shorter."""
    import ctypes as C
    c = build_decode_case(2480, [777], 1, 4, 128, 16)
    cache = c["cache"]
    dev = cache.phys.device
    need = 25088                                         # header 256 + tickets 16384 + lse 256 + partials 2 * 8 * 128 * 4
    buf = torch.full((need + 4096,), 0xA5, dtype=torch.uint8, device=dev)
    buf[:need] = 0
    q = bf16_tensor(c["q"])
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    bt, sl, qsl = (torch.from_numpy(c[k]).to(dev) for k in ("bt", "seq_lens", "qsl"))
    gk, gv = torch.from_numpy(c["gk"]).to(dev), torch.from_numpy(c["gv"]).to(dev)
    st = (C.c_int64 * 6)(*cache.strides)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731

    def call(nbytes):
        return _lib.load().hkv_decode(p(q), *(p(t) for t in cache.flat), st, cache.PS, p(bt), bt.shape[1], p(sl), p(qsl),
                                      1, 1, 4, 128, 1, c["sm"], 1.0, p(gk), p(gv), p(buf), nbytes, 1, p(out),
                                      C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert call(need - 1) == -5
    assert call(need) == 0
    torch.cuda.synchronize()
    assert (buf[need:] == 0xA5).all()
    assert_close(out, oracle_decode(c))


@pytest.mark.parametrize("D", [128, 256])
def test_pieces_in_which_some_rows_see_no_key(D):
    """one long sequence on a grid that gives (nearly) every unit its own partition, eight query tokens on one head: the
    last unit holds three tokens, which only the last three query tokens may see, so for the other rows that piece is
    empty (log-sum-exp -inf, its partial must be ignored by the merge); plus a request whose context is shorter than its
    query tokens, whose first rows see nothing at all and must come out as zeros"""
    UT = 32                                              # tokens of a unit of the stream
    sms = K.num_sms()
    n_units = sms * (3 if D == 128 else 2) - 12 - 2      # about one unit per partition (a sequence weighs its units + 12)
    lens = [UT * n_units + 3, 5]
    c = build_decode_case(2700 + D, lens, 1, 1, D, 16, ql_list=[8, 8])
    ref = oracle_decode(c)
    out, ws = gpu_decode(c, qlmax=8)
    assert K.workspace_status(ws) == 0
    got = out.float().cpu().numpy()
    q1 = int(c["qsl"][1])
    # request 1: context 5, 8 query tokens: token t sees 5 - 8 + t + 1 keys, none for t < 3
    assert (got[q1:q1 + 3] == 0).all()
    ref2 = ref.copy()
    ref2[q1:q1 + 3] = 0.0                                        # (the oracle leaves rows without keys as NaN or zero)
    assert_close(out, np.nan_to_num(ref2, nan=0.0))
    o2, _ = gpu_decode(c, ws=ws, qlmax=8)
    assert torch.equal(out, o2)
