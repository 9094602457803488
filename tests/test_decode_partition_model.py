"""The bookkeeping of the balanced decode partition (csrc/ktk_decode_stream.cu), restated in Python.

The kernel cuts the concatenated page lists into equal chunks, one per CTA; a CTA writes the output of a
list it sees whole, or a partial into its "tail" slot (the list starts here and goes on) or its "head" slot
(the list started earlier); the combine pass of CTA c merges the list that starts in c and continues.  This
model runs the same rules on the host and checks the invariants the kernels rely on: every entry is read by
exactly one CTA, every list gets exactly one writer of its output, every slot written is read exactly once.
(The kernels themselves are checked against the oracle in the GPU tests.)
"""
import random


def _walk(units, total, chunk, grid):
    """units: list of (key, start, length, count) in position order.  Returns (outputs, slots, covered)."""
    covered = {k: [0] * cnt for k, _, _, cnt in units}
    out, slots = {}, {}
    for c in range(grid):
        p0, p1 = c * chunk, min((c + 1) * chunk, total)
        if p1 <= p0:
            continue
        for key, start, length, cnt in units:
            if start + length <= p0 or start >= p1 or length == 0:
                continue
            lo, hi = max(p0 - start, 0), min(p1 - start, length)
            first = p0 <= start
            e_lo, e_hi = min(lo, cnt), min(hi, cnt)
            whole = first and e_hi == cnt
            partial = (not whole) and (first or e_hi > e_lo)
            for e in range(e_lo, e_hi):
                covered[key][e] += 1
            if whole:
                assert key not in out
                out[key] = "direct"
            elif partial:
                slot = (c, 1 if first else 0)
                assert slot not in slots and e_hi > e_lo
                slots[slot] = (key, e_lo, e_hi)
    for c in range(grid):                                    # the combine pass
        p0, p1 = c * chunk, min((c + 1) * chunk, total)
        if p1 <= p0 or p1 >= total:
            continue
        key, start, length, cnt = next(u for u in units if u[1] <= p1 - 1 < u[1] + u[2])
        if start < p0 or start + cnt <= p1:
            continue
        pieces, c2 = [], c
        while c2 * chunk < start + cnt:
            k2, a, b = slots.pop((c2, 1 if c2 == c else 0))
            assert k2 == key
            pieces.append((a, b))
            c2 += 1
        pieces.sort()
        assert pieces[0][0] == 0 and pieces[-1][1] == cnt
        assert all(pieces[i][1] == pieces[i + 1][0] for i in range(len(pieces) - 1))
        assert key not in out
        out[key] = "combined"
    return out, slots, covered


def test_padded_rows():
    rng = random.Random(1)
    for _ in range(1500):
        U, wmax = rng.randint(1, 40), rng.randint(1, 70)
        cnts = [rng.choice([0, wmax, rng.randint(0, wmax)]) for _ in range(U)]
        total = U * wmax
        grid = min(rng.choice([1, 2, 3, 7, 16, 444]), max(1, -(-total // rng.choice([1, 4, 16]))))
        chunk = -(-total // grid)
        grid = -(-total // chunk)
        units = [(u, u * wmax, wmax, cnts[u]) for u in range(U)]
        out, slots, covered = _walk(units, total, chunk, grid)
        assert not slots and len(out) == U
        assert all(all(x == 1 for x in cv) for cv in covered.values())


def test_csr_entries():
    rng = random.Random(2)
    for _ in range(1500):
        B, hkv = rng.randint(1, 12), rng.choice([1, 2, 8])
        ns = [rng.choice([0, 0, 1, rng.randint(1, 90)]) for _ in range(B)]
        units, pos = [], 0
        for b, n in enumerate(ns):
            for h in range(hkv):
                units.append(((b, h), pos, n, n))
                pos += n
        total = pos
        grid = rng.choice([1, 2, 5, 17, 444])
        chunk = max(-(-total // grid), rng.choice([1, 4, 16])) if total else 16
        out, slots, covered = _walk(units, total, chunk, grid)
        assert not slots
        assert all(all(x == 1 for x in cv) for cv in covered.values())
        # lists without entries own no position: the combine pass writes their zero rows separately
        assert set(out) == {k for k, _, n, _ in units if n > 0}
