"""Host-side model of count-in protocols for the fused GEMM -> reduce-scatter kernel
(csrc/kernels/tp_gemm.cu).  Every CTA pair walks its tiles in the kernel's order (peers'
rows first, own rows last), sends a partial tile to its owner and counts it in, and may
only finish an own tile once all peers have counted theirs in.  The kernel counts a tile in
at once.  A variant that counted in ONE TILE LATER (to hide the NVLink round trip) was
tried on GPUs: it completed with 2 ranks and timed out with 8.  This model shows why --
ranks wait on each other round the ring while holding each other's counts -- and that
delivering the pending count before the wait restores progress; it guards any future
attempt at deferral."""
import pytest


def tile_coords(n, rank, tile, tilesN, M, TM, groupRows):
    blocks = M // TM; bpr = blocks // n; tilesPerRank = bpr * tilesN
    r, w = divmod(tile, tilesPerRank)
    perGroup = groupRows * tilesN
    g, wg = divmod(w, perGroup)
    gsize = min(groupRows, bpr - g * groupRows)
    tn = wg // gsize
    rb = r * bpr + g * groupRows + (wg - tn * gsize)
    rb = (rb + (rank + 1) * bpr) % blocks
    return rb, tn
def run(n, flush_before_wait, M=8192, N=8192, TM=256, BN=256, units=74, groupRows=8):
    blocks = M // TM; bpr = blocks // n; tilesN = N // BN; nTiles = blocks * tilesN
    need = (n - 1) * tilesN
    count = [[0] * bpr for _ in range(n)]
    seqs = {(r, u): [tile_coords(n, r, t, tilesN, M, TM, groupRows) for t in range(u, nTiles, units)] for r in range(n) for u in range(units)}
    pos = {k: 0 for k in seqs}; pend = {k: None for k in seqs}; done = set()
    def deliver(k):
        if pend[k] is not None:
            o, rb = pend[k]; count[o][rb] += 1; pend[k] = None
    progress = True
    while progress and len(done) < len(seqs):
        progress = False
        for k, seq in seqs.items():
            if k in done: continue
            r = k[0]
            while pos[k] < len(seq):
                rb, tn = seq[pos[k]]; owner = rb // bpr
                if owner == r:
                    if flush_before_wait and pend[k] is not None:
                        deliver(k); progress = True
                    if count[r][rb - r * bpr] < need: break
                deliver(k)
                if owner != r: pend[k] = (owner, rb - owner * bpr)
                pos[k] += 1; progress = True
            if pos[k] == len(seq):
                deliver(k); done.add(k); progress = True
    return len(done) == len(seqs)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("shape", [(8192, 8192), (4096, 8192), (8192, 2048)])
def test_count_in_protocol_makes_progress(n, shape):
    M, N = shape
    assert run(n, True, M=M, N=N)


def test_the_model_reproduces_the_circular_wait_of_the_unflushed_variant():
    assert run(2, False)
    assert not run(4, False)
    assert not run(8, False)
