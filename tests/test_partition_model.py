"""CPU model of the decode kernel's stream decomposition (horizon_kernels_b200/csrc/hkv_decode.cu): every (request, kv
head) sequence counts as PIECE_COST cost slots followed by its units; the concatenation is cut into equal partitions;
a partition's piece of a sequence is the part of the sequence's UNITS inside the partition. The model restates the
kernel's integer arithmetic (unit count of a partition, piece extents, the slot a partial piece is stored in, the
ticket counter a split sequence uses) and checks the invariants the in-kernel log-sum-exp merge relies on."""
import numpy as np
import pytest


def wt(U, PC):
    return U + PC if U > 0 else 0


def units_before(x, S, U, W, KVH, PC):
    """units of a request (weighted start S, KVH sequences of weight W = U + PC) that lie before stream position x"""
    if W == 0 or x <= S:
        return 0
    t = min(x - S, KVH * W)
    return (t // W) * U + max(0, t % W - PC)


def decompose(Us, KVH, PC, n_parts):
    """-> per partition: list of pieces (b, h, blk0, n, complete, first_part, first_slot) and the unit count"""
    Ws = [wt(U, PC) for U in Us]
    total = sum(Ws) * KVH
    per = max(1, -(-total // n_parts))
    starts = np.concatenate([[0], np.cumsum([W * KVH for W in Ws])])
    parts = []
    for part in range(n_parts):
        lo, hi = part * per, min(total, (part + 1) * per)
        pieces, n_units = [], 0
        if lo < hi:
            n_units = sum(units_before(hi, int(starts[b]), Us[b], Ws[b], KVH, PC)
                          - units_before(lo, int(starts[b]), Us[b], Ws[b], KVH, PC) for b in range(len(Us)))
            for b, (U, W) in enumerate(zip(Us, Ws)):
                for h in range(KVH if W else 0):
                    seq0 = int(starts[b]) + h * W
                    u0, end = seq0 + PC, seq0 + W
                    p_lo, p_hi = max(lo, u0), min(hi, end)
                    if p_lo >= p_hi:
                        continue
                    first_part = u0 // per
                    first_slot = 0 if first_part * per >= seq0 else 1
                    pieces.append((b, h, p_lo - u0, p_hi - p_lo, p_lo == u0 and p_hi == end, first_part, first_slot))
        parts.append((pieces, n_units))
    return parts, per


@pytest.mark.parametrize("seed", range(12))
def test_weighted_partitions_cover_every_unit_once_and_keep_the_slot_invariants(seed):
    rng = np.random.default_rng(seed)
    B = int(rng.integers(1, 70))
    KVH = int(rng.choice([1, 2, 8]))
    PC = int(rng.choice([0, 4, 8, 12]))
    n_parts = int(rng.choice([1, 7, 64, 444]))
    Us = [int(x) for x in np.maximum(0, np.exp(rng.uniform(0, 7, B)).astype(int) - rng.integers(0, 2, B) * 3)]
    if sum(Us) == 0:
        Us[0] = 5
    parts, per = decompose(Us, KVH, PC, n_parts)
    covered = {}
    for part, (pieces, n_units) in enumerate(parts):
        assert n_units == sum(p[3] for p in pieces)                      # the closed form equals the walk
        partial = [p for p in pieces if not p[4]]
        assert len(partial) <= 2                                         # two workspace slots per partition suffice
        for i, (b, h, blk0, n, complete, first_part, first_slot) in enumerate(pieces):
            for u in range(blk0, blk0 + n):
                assert (b, h, u) not in covered
                covered[(b, h, u)] = part
            if not complete:
                assert i == 0 or i == len(pieces) - 1                    # only the first and the last piece can be partial
                if blk0 == 0:                                            # the sequence starts here: its stored slot
                    assert first_part == part
                    assert first_slot == (0 if i == 0 else 1)
                else:                                                    # a continuation is the partition's first piece
                    assert i == 0 and first_part < part
    assert len(covered) == sum(Us) * KVH
    # a split sequence occupies first_part .. last partition without gaps; the closed forms the ticket round uses
    # (first = u0 // per, last = (u0 + U - 1) // per, pieces = last - first + 1) name exactly those partitions, and no
    # two split sequences share a ticket counter (the counter's index is the sequence's last partition)
    Ws = [wt(U, PC) for U in Us]
    starts = np.concatenate([[0], np.cumsum([W * KVH for W in Ws])])
    ticket_owner = {}
    for b, U in enumerate(Us):
        for h in range(KVH if U else 0):
            ps = sorted({covered[(b, h, u)] for u in range(U)})
            assert ps == list(range(ps[0], ps[-1] + 1))
            u0 = int(starts[b]) + h * Ws[b] + PC
            first, last = u0 // per, (u0 + U - 1) // per
            assert (first, last) == (ps[0], ps[-1])
            if first != last:
                assert last not in ticket_owner
                ticket_owner[last] = (b, h)
                # the piece in `last` is that partition's first piece (slot 0), as are those of the partitions between
                for part in range(first + 1, last + 1):
                    assert parts[part][0][0][:2] == (b, h)
