"""Work split of the streaming GEMV kernel (qf_gemv_slab.cu), restated on the CPU.

Thread block i of G owns the units [i*U/G, (i+1)*U/G); a row block (K/128 consecutive units) that spans several
thread blocks is finished by the one that holds its last unit (the owner), which adds the partial sums the others
left in the workspace. The checks: every unit is covered exactly once, the closed form the kernel uses to find the
first contributor is right, every split row block has exactly one owner, the owner meets it as its FIRST segment
and every other contributor as its LAST one (so one workspace slot per thread block suffices), and an owner only
waits for thread blocks with a lower index.
"""
import pytest


def cta_of(u, U, G):
    return ((u + 1) * G - 1) // U


def segments(i, U, G, chunks):
    """What thread block i does, as the kernel's consumer loop decides it: (kind, row_block, c_lo, c_hi)."""
    u0, u1 = i * U // G, (i + 1) * U // G
    out = []
    b, c = divmod(u0, chunks)
    c_lo = c
    for it in range(u1 - u0):
        c += 1
        if c == chunks or it == u1 - u0 - 1:
            if c_lo == 0 and c == chunks:
                out.append(("full", b, c_lo, c))
            elif c == chunks:
                out.append(("owner", b, c_lo, c))
            else:
                out.append(("contrib", b, c_lo, c))
            if c == chunks:
                c = 0
                b += 1
            c_lo = c
    return out


@pytest.mark.parametrize("blocks,chunks,G", [
    (64, 32, 148), (64, 32, 296), (64, 32, 444), (224, 32, 444), (64, 112, 296), (16, 8, 128), (16, 8, 100),
    (1, 8, 8), (1, 8, 3), (3, 1, 3), (5, 7, 11), (896, 64, 592), (128, 64, 148), (20, 64, 592), (2, 4, 1),
    (8, 32, 7), (48, 64, 148), (80, 32, 148), (112, 32, 148), (148, 32, 148), (224, 224, 592),
])
def test_partition_and_ownership(blocks, chunks, G):
    U = blocks * chunks
    G = min(G, U)
    covered = [0] * U
    for i in range(G):
        u0, u1 = i * U // G, (i + 1) * U // G
        assert u1 > u0
        for u in range(u0, u1):
            covered[u] += 1
            assert cta_of(u, U, G) == i
    assert covered == [1] * U

    per_block = {}
    for i in range(G):
        segs = segments(i, U, G, chunks)
        kinds = [k for (k, *_rest) in segs]
        # at most one owner segment, and it comes first; at most one contributor segment, and it comes last
        assert kinds.count("owner") <= 1 and kinds.count("contrib") <= 1
        if "owner" in kinds:
            assert kinds[0] == "owner"
        if "contrib" in kinds:
            assert kinds[-1] == "contrib"
        for (k, b, c_lo, c_hi) in segs:
            per_block.setdefault(b, []).append((i, k, c_lo, c_hi))

    assert sorted(per_block) == list(range(blocks))
    for b, parts in per_block.items():
        parts.sort()
        # the pieces tile [0, chunks) in thread-block order
        pos = 0
        for (_i, _k, c_lo, c_hi) in parts:
            assert c_lo == pos and c_hi > c_lo
            pos = c_hi
        assert pos == chunks
        if len(parts) == 1:
            assert parts[0][1] == "full"
            continue
        owner = parts[-1]
        assert owner[1] == "owner"
        assert all(k == "contrib" for (_i, k, _a, _b) in parts[:-1])
        ids = [i for (i, *_r) in parts]
        # the kernel's formula for the first contributor, and contributors = every block from there to owner - 1
        assert ids[0] == cta_of(b * chunks, U, G)
        assert ids == list(range(ids[0], owner[0] + 1))
