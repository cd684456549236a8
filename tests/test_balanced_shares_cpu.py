"""The arithmetic of the balanced work distribution (host functions of the C ABI): shares tile the
list exactly, the owner function inverts the begin function, and a walk over every CTA's share
with the kernel's slot rule (sequence * head groups + head group + CTA) writes every partial slot
at most once and leaves, for every (sequence, head group), exactly the slots the merge will read."""
import random

from wsvd_b200 import _lib

TILE = 128


def _walk(lens, n_hg, n_ctas):
    lib = _lib.lib()
    tiles = [(n + TILE - 1) // TILE if n > 0 else 0 for n in lens]
    prefix = [0]
    for t in tiles:
        prefix.append(prefix[-1] + t)
    total = prefix[-1] * n_hg
    shares = min(n_ctas, total)
    written = {}
    for c in range(shares):
        begin, end = lib.wsvd_share_begin(c, total, shares), lib.wsvd_share_begin(c + 1, total, shares)
        assert end > begin, "no share is empty"
        b = max(i for i in range(len(lens)) if prefix[i] * n_hg <= begin and tiles[i] > 0)
        rem = begin - prefix[b] * n_hg
        hg, t, left = rem // tiles[b], rem % tiles[b], end - begin
        while left > 0:
            seg = min(left, tiles[b] - t)
            slot = b * n_hg + hg + c
            assert slot not in written and slot < len(lens) * n_hg + n_ctas
            written[slot] = (b, hg, t, t + seg)
            left, t, hg = left - seg, 0, hg + 1
            if hg == n_hg:
                hg, b = 0, b + 1
                while b < len(lens) and tiles[b] == 0:
                    b += 1
    for b, nt in enumerate(tiles):
        for hg in range(n_hg if nt else 0):
            first = prefix[b] * n_hg + hg * nt
            c0, c1 = lib.wsvd_share_owner(first, total, shares), lib.wsvd_share_owner(first + nt - 1, total, shares)
            cover = [written[b * n_hg + hg + c] for c in range(c0, c1 + 1)]
            assert all(w[:2] == (b, hg) for w in cover)
            assert cover[0][2] == 0 and cover[-1][3] == nt
            assert all(x[3] == y[2] for x, y in zip(cover, cover[1:]))
    return total, shares


def test_owner_inverts_begin():
    lib = _lib.lib()
    rng = random.Random(1)
    for _ in range(300):
        total, n = rng.randint(1, 5000), rng.randint(1, 300)
        n = min(n, total)
        for tile in rng.sample(range(total), min(total, 50)):
            c = lib.wsvd_share_owner(tile, total, n)
            assert 0 <= c < n and lib.wsvd_share_begin(c, total, n) <= tile < lib.wsvd_share_begin(c + 1, total, n)
    assert lib.wsvd_share_begin(0, 10, 4) == 0 and lib.wsvd_share_begin(4, 10, 4) == 10


def test_benchmark_shapes_and_edge_cases():
    assert _walk([8192] * 16, 10, 148) == (10240, 148)
    assert _walk([1500, 0, 257, 0, 2049], 2, 148) == (64, 64)
    assert _walk([1], 1, 148) == (1, 1)
    assert _walk([0, 0, 129, 128, 1, 0, 4000, 127], 2, 7)[1] == 7


def test_random_ragged_batches():
    rng = random.Random(2)
    for _ in range(300):
        lens = [rng.choice([0, 1, 127, 128, 129, rng.randint(1, 5000)]) for _ in range(rng.randint(1, 40))]
        if sum(lens) == 0:
            continue
        _walk(lens, rng.randint(1, 10), rng.randint(1, 200))
