"""The decode configurations of the benchmark at their FULL sizes (batch 64 with contexts in [1024, 8192]; batch 8 at
131,072 tokens; the 2048-request hybrid batch at head_dim 256, whose page pool passes 4 GiB), where a CPU pass over the
whole batch would take minutes. Checked through what does not depend on the size:

  * a sample of requests (the longest, the shortest, one in between) against the oracle over the same cache bytes, their
    pages gathered into a small pool;
  * placement: the same tokens written to other physical pages decode to the same bits;
  * scales: twice the global value scale, or twice the output scale, doubles every output exactly (powers of two pass
    through fp32 products and the bf16 rounding unchanged), and twice the global key scale with half the softmax scale
    changes nothing.

The cache is filled on the device by the write kernel, whose bytes the write tests pin to the oracle."""
import math

import numpy as np
import pytest
import torch

from cases import assert_close, bf16_bits
from horizon_kernels_b200 import kernels as K
from horizon_kernels_b200 import layout as Lt
from oracle import kvfp4 as O

pytestmark = pytest.mark.gpu
PS = 16
CHUNK = 8192                    # pages written per launch of the fill


def draw_lens(law, B, seed):
    rng = np.random.default_rng(seed)
    if law[0] == "const":
        return [law[1]] * B
    if law[0] == "loguniform":
        return [int(round(math.exp(x))) for x in rng.uniform(math.log(law[1]), math.log(law[2]), B)]
    return [int(x) for x in rng.integers(law[1], law[2] + 1, B)]


class Filled:
    """a page pool holding seeded K / V of the given context lengths at a seeded random placement"""

    def __init__(self, lens, KVH, D, data_seed, place_seed, slack):
        dev = "cuda"
        self.lens, self.KVH, self.D = lens, KVH, D
        pages = [(n + PS - 1) // PS for n in lens]
        tot, MP = sum(pages), max(pages)
        NP = tot + int(tot * slack) + 8
        self.phys = torch.full((NP, 2 * KVH, PS, Lt.slot_bytes(D)), 0x7F, dtype=torch.uint8, device=dev)
        self.flat, self.strides = Lt.flat_views(*Lt.slot_views(self.phys, KVH, D))
        g = torch.Generator(device=dev).manual_seed(place_seed)
        perm = torch.randperm(NP, generator=g, device=dev)[:tot]
        self.bt = torch.zeros((len(lens), MP), dtype=torch.int32, device=dev)
        o = 0
        for b, n in enumerate(pages):
            self.bt[b, :n] = perm[o:o + n].to(torch.int32)
            o += n
        self.pages = pages
        # per-tensor scales of the configurations: amax / (6 * 448) with the outlier channels at about 20 x 4.5 sigma
        self.gk = torch.full((KVH,), 100.0 / (6 * 448), device=dev)
        self.gv = torch.full((KVH,), 5.5 / (6 * 448), device=dev)
        ch = [3, D // 4 + 3, D // 2 + 3, 3 * D // 4 + 3]
        for i in range(0, tot, CHUNK):
            pg = perm[i:i + CHUNK]
            n = pg.numel() * PS
            gd = torch.Generator(device=dev).manual_seed(data_seed * 100003 + i)   # the data do not depend on the place
            k = torch.randn(n, KVH, D, generator=gd, device=dev)
            k[:, :, ch] *= 20
            v = torch.randn(n, KVH, D, generator=gd, device=dev)
            sl = (pg[:, None] * PS + torch.arange(PS, device=dev)[None, :]).reshape(-1)
            K.write(k.to(torch.bfloat16), v.to(torch.bfloat16), self.flat, self.strides, PS, sl, self.gk, self.gv, True)
            del k, v
        self.sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        self.qsl = torch.arange(len(lens) + 1, dtype=torch.int32, device=dev)

    def decode(self, q, ws, sm=None, v_scale=1.0, gk=None, gv=None):
        out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
        K.decode_ragged(q, self.flat, self.strides, PS, self.bt, self.sl, self.qsl,
                        self.D ** -0.5 if sm is None else sm, v_scale, self.gk if gk is None else gk,
                        self.gv if gv is None else gv, 1, out, ws)
        assert K.workspace_status(ws) == 0
        return out

    def oracle_sample(self, q, rows, v_scale=1.0):
        """fp64 attention of the oracle for the requests `rows`, over a pool holding only their pages"""
        idx = torch.cat([self.bt[b, :self.pages[b]].long() for b in rows])
        sub = self.phys[idx].cpu().numpy().reshape(-1)
        MP = max(self.pages[b] for b in rows)
        bt = np.zeros((len(rows), MP), np.int32)
        o = 0
        for i, b in enumerate(rows):
            bt[i, :self.pages[b]] = np.arange(o, o + self.pages[b])
            o += self.pages[b]
        lens = np.array([self.lens[b] for b in rows], np.int32)
        qb = bf16_bits(q[rows])
        ref, _ = O.attention(qb, sub, O.Layout.slots(PS, self.KVH, self.D), bt, lens,
                             np.arange(len(rows) + 1, dtype=np.int32), self.KVH, self.D ** -0.5,
                             self.gk.cpu().numpy(), self.gv.cpu().numpy(), v_scale)
        return ref


FULL = [
    # name, batch, query heads, kv heads, head_dim, length law, pool slack, requests sampled for the oracle
    ("batch64_1k_8k", 64, 32, 8, 128, ("uniform", 1024, 8192), 0.25, 3),
    ("batch8_128k", 8, 64, 8, 128, ("const", 131072), 0.0, 1),
    ("hybrid2048_d256", 2048, 16, 2, 256, ("loguniform", 128, 32768), 0.25, 3),
]


@pytest.mark.parametrize("name,B,HQ,KVH,D,law,slack,n_sample", FULL, ids=[f[0] for f in FULL])
def test_full_size_properties(name, B, HQ, KVH, D, law, slack, n_sample):
    lens = draw_lens(law, B, 20261125)
    G = HQ // KVH
    a = Filled(lens, KVH, D, data_seed=11, place_seed=1, slack=slack)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, HQ, D, generator=g, device="cuda").to(torch.bfloat16)
    ws = K.alloc_workspace(B, KVH, G, D, 1, "cuda")
    out = a.decode(q, ws)
    assert bool(torch.isfinite(out.float()).all())

    # a sample of requests against the oracle
    order = sorted(range(B), key=lambda b: lens[b])
    rows = [order[-1]] if n_sample == 1 else sorted({order[-1], order[0], order[B // 2]})
    ref = a.oracle_sample(q, rows)
    mx, mn, rl = assert_close(out[rows], ref, name)
    print(f"{name}: requests {rows} of lengths {[lens[b] for b in rows]}: max-abs {mx:.3e} mean-abs {mn:.3e} "
          f"rel-l2 {rl:.3e}")

    # scales that are powers of two pass through exactly
    two = a.decode(q, ws, gv=a.gv * 2)
    assert torch.equal(two.float(), out.float() * 2)
    two = a.decode(q, ws, v_scale=2.0)
    assert torch.equal(two.float(), out.float() * 2)
    same = a.decode(q, ws, gk=a.gk * 2, sm=0.5 * D ** -0.5)
    assert torch.equal(same, out)

    # the same tokens at other physical pages
    flat_a = a.phys
    b = Filled(lens, KVH, D, data_seed=11, place_seed=2, slack=slack)
    assert not torch.equal(a.bt, b.bt)
    r = rows[0]
    pa, pb = a.bt[r, :a.pages[r]].long(), b.bt[r, :b.pages[r]].long()
    assert torch.equal(flat_a[pa], b.phys[pb])                      # same page contents, different places
    del flat_a
    out_b = b.decode(q, ws)
    assert torch.equal(out_b, out)
