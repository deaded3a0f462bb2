"""The ordering protocol of the fused two-launch kernel (csrc/pair_fft.cuh), replayed on the CPU.

A persistent grid draws tickets from one work list ([first-launch tiles of chunk j][last-launch
tiles of chunk j - lag] per super-step; a block draws its next ticket while it works on the current
one); the intermediate of chunk c lives in ring slot c mod R; two counters per
chunk order the ring; a tile's signal is deferred into the block's next tile unless the block has
to wait.  The model below mirrors the kernel's control flow step by step and lets a seeded
adversarial scheduler pick which block moves next.  Checked for every interleaving tried:
  * progress: some block can always move until all items are done (no deadlock),
  * a last-launch tile only reads a slot when every first-launch tile of ITS chunk has stored there,
  * a first-launch tile only overwrites a slot when every last-launch tile of the slot's previous
    chunk has read it.
"""
import random

import pytest

R = 4  # ring chunks, as in tfft_plan_fuse_launches


class Block:
    def __init__(self):
        self.item = None        # (is_first, chunk, local_tile) of the current ticket, None when the list is exhausted
        self.next = None        # the ticket drawn ahead (an index into the list), None before the draw
        self.phase = "check"    # check -> (wait) -> load -> hook -> store
        self.pending = None     # counter key of the finished, unpublished tile
        self.exhausted = False


def run_model(n_signals_tiles1, n_signals_tiles2, batch, chunk_signals, lag, grid, seed):
    """n_signals_tiles{1,2}: tiles per signal of the first / last launch."""
    rng = random.Random(seed)
    n_chunks = (batch + chunk_signals - 1) // chunk_signals
    t1, t2 = n_signals_tiles1 * chunk_signals, n_signals_tiles2 * chunk_signals
    n_tiles1, n_tiles2 = n_signals_tiles1 * batch, n_signals_tiles2 * batch

    def tiles_in(chunk, per, total):
        return min(per, total - chunk * per)

    # the work list, exactly as the kernel decodes item i (None: an empty slot, skipped with a fresh draw)
    per = t1 + t2
    items = []
    for i in range((n_chunks + lag) * per):
        j, slot = divmod(i, per)
        is_first = slot < t1
        chunk = j if is_first else j - lag
        local = slot if is_first else slot - t1
        if chunk < 0 or chunk >= n_chunks or chunk * (t1 if is_first else t2) + local >= (n_tiles1 if is_first else n_tiles2):
            items.append(None)
        else:
            items.append((is_first, chunk, local))
    queue = [0]

    def draw():
        queue[0] += 1
        return queue[0] - 1

    def take(b, ticket):
        """The block starts the iteration of `ticket`: skips empty slots as the kernel does."""
        while ticket < len(items) and items[ticket] is None:
            ticket = draw()
        if ticket >= len(items):
            b.item, b.exhausted = None, True
        else:
            b.item = items[ticket]
        b.next = None
        b.phase = "check"

    blocks = [Block() for _ in range(grid)]
    for b in blocks:
        take(b, draw())

    done = {}                                  # published counters: ("first"|"last", chunk) -> tiles
    stored = [dict() for _ in range(R)]        # ring slot -> {local first-launch tile: chunk}
    reads = {}                                 # chunk -> last-launch tiles that have read their slot
    finished = 0
    total = sum(1 for it in items if it is not None)

    def dependency(is_first, chunk):
        if is_first:
            if chunk < R:
                return None
            dep = chunk - R
            return ("last", dep), tiles_in(dep, t2, n_tiles2)
        return ("first", chunk), tiles_in(chunk, t1, n_tiles1)

    def runnable(b):
        if b.exhausted:
            return b.pending is not None  # the final publish after the loop
        if b.phase != "wait":
            return True
        key, need = dependency(*b.item[:2])
        return done.get(key, 0) >= need

    steps = 0
    while True:
        live = [b for b in blocks if runnable(b)]
        if not live:
            break
        b = rng.choice(live)
        steps += 1
        if b.exhausted:
            done[b.pending] = done.get(b.pending, 0) + 1
            b.pending = None
            continue
        is_first, chunk, local = b.item
        dep = dependency(is_first, chunk)
        if b.phase == "check":
            if dep and done.get(dep[0], 0) < dep[1]:
                if b.pending is not None:  # a block that waits holds no unpublished tile
                    done[b.pending] = done.get(b.pending, 0) + 1
                    b.pending = None
                b.phase = "wait"
            else:
                b.phase = "load"
        elif b.phase == "wait":
            b.phase = "load"
        elif b.phase == "load":
            if not is_first:
                slot = stored[chunk % R]
                want = tiles_in(chunk, t1, n_tiles1)
                assert sum(1 for v in slot.values() if v == chunk) == want, "read before the chunk was complete"
                reads[chunk] = reads.get(chunk, 0) + 1
            b.phase = "hook"
        elif b.phase == "hook":
            if b.pending is not None:
                done[b.pending] = done.get(b.pending, 0) + 1
                b.pending = None
            b.next = draw()  # the next ticket is drawn while this tile runs
            b.phase = "store"
        else:
            if is_first:
                if chunk >= R:
                    prev = chunk - R
                    assert reads.get(prev, 0) == tiles_in(prev, t2, n_tiles2), "slot overwritten before it was read"
                stored[chunk % R][local] = chunk
            b.pending = ("first" if is_first else "last", chunk)
            finished += 1
            take(b, b.next)
    assert finished == total, f"deadlock after {steps} steps: {finished} of {total} items"
    for c in range(n_chunks):
        assert done.get(("first", c), 0) == tiles_in(c, t1, n_tiles1)
        assert done.get(("last", c), 0) == tiles_in(c, t2, n_tiles2)


@pytest.mark.parametrize("lag", [0, 1, 2])
@pytest.mark.parametrize("batch,chunk_signals,grid", [(1, 1, 3), (5, 2, 4), (9, 1, 7), (13, 4, 16), (32, 2, 5), (23, 2, 64)])
def test_schedule_makes_progress_and_orders_the_ring(lag, batch, chunk_signals, grid):
    for seed in range(6):
        run_model(4, 2, batch, chunk_signals, lag, grid, seed)
        run_model(1, 3, batch, chunk_signals, lag, grid, 100 + seed)
