"""Exhaustive interleaving check of the peer-memory flag protocols (host-side model, no GPU).

The fused collectives synchronise ranks through counters / epoch flags in symmetric memory and reuse two staging
regions ("parities") alternately.  Their safety argument: a rank cannot finish call c before every peer has started
call c, so no rank is ever more than one call ahead and two regions suffice.  This test enumerates every
interleaving of the ranks' steps for a few calls and checks that
  * a reader only ever sees data of the call it is executing (no stale and no premature overwrite),
  * arrival counters never exceed the world size and are zero again when all ranks are done.
A deliberately broken variant (one region instead of two) must be caught, which shows the checker can fail.
"""

def _explore(initial, step_fn, done_fn, check_final):
    """Depth-first search over all interleavings.  ``step_fn(state, rank)`` returns the successor state, None when
    the rank is blocked or finished, or raises AssertionError on a violation."""
    seen, stack, finals = {initial}, [initial], 0
    world = len(initial[0])
    while stack:
        st = stack.pop()
        progressed = False
        for r in range(world):
            nxt = step_fn(st, r)
            if nxt is None:
                continue
            progressed = True
            if nxt not in seen:
                seen.add(nxt)
                stack.append(nxt)
        if not progressed:
            assert done_fn(st), f"deadlock in state {st}"
            check_final(st)
            finals += 1
    return len(seen), finals


# -----------------------------------------------------------------------------------------------------------------
# one-shot all-reduce with a staged input: per call c (region c % regions)
#   0            write own staging region
#   1 .. W       bump the call's counter on every rank (self included)
#   W + 1        wait until the own counter shows W arrivals
#   W + 2        reset the own counter (a plain store in the kernel, hence its own step)
#   W + 3 .. 2W+2  read every rank's staging region: must hold call c
# state = (pcs, calls, counters[rank][region], stage[rank][region])
# -----------------------------------------------------------------------------------------------------------------
def _allreduce_model(world, calls, regions):
    def step(st, r):
        pcs, cs, cnt, stage = st
        c, pc = cs[r], pcs[r]
        if c == calls:
            return None
        reg = c % regions
        cnt_l, stage_l = [list(x) for x in cnt], [list(x) for x in stage]
        if pc == 0:
            stage_l[r][reg] = c
        elif 1 <= pc <= world:
            p = pc - 1
            cnt_l[p][reg] += 1
            assert cnt_l[p][reg] <= world, f"counter overflow at rank {p}: {st}"
        elif pc == world + 1:
            if cnt[r][reg] < world:
                return None
        elif pc == world + 2:
            cnt_l[r][reg] = 0
        else:
            p = pc - (world + 3)
            assert stage[p][reg] == c, f"rank {r} call {c} read call {stage[p][reg]} from rank {p}"
        pc += 1
        pcs_l, cs_l = list(pcs), list(cs)
        if pc == 2 * world + 3:
            pc, cs_l[r] = 0, c + 1
        pcs_l[r] = pc
        return (tuple(pcs_l), tuple(cs_l), tuple(tuple(x) for x in cnt_l), tuple(tuple(x) for x in stage_l))

    init = (tuple([0] * world), tuple([0] * world), tuple(tuple([0] * regions) for _ in range(world)),
            tuple(tuple([-1] * regions) for _ in range(world)))

    def final(st):
        assert all(v == 0 for row in st[2] for v in row), f"counters not clean: {st[2]}"
    return init, step, (lambda st: all(c == calls for c in st[1])), final


def test_allreduce_two_regions_are_enough():
    for world, calls in ((2, 4), (3, 3)):
        init, step, done, final = _allreduce_model(world, calls, regions=2)
        states, finals = _explore(init, step, done, final)
        assert states > 100 and finals >= 1


def test_allreduce_one_region_is_caught():
    init, step, done, final = _allreduce_model(2, 3, regions=1)
    try:
        _explore(init, step, done, final)
    except AssertionError:
        return
    raise AssertionError("the single-region protocol should have shown a stale read or a counter overflow")


# -----------------------------------------------------------------------------------------------------------------
# all-gather in front of a GEMM (push model, epoch flags): per call c (region c % regions, epoch c + 1)
#   0 .. W-1     store own rows into every rank's gathered buffer
#   W .. 2W-1    publish the epoch in slot `me` of every rank's flag array
#   2W .. 3W-1   for each source q: wait flag[q] >= epoch, then read rows q: must hold call c
# state = (pcs, calls, flags[rank][region][src], data[rank][region][src])
# -----------------------------------------------------------------------------------------------------------------
def _allgather_model(world, calls, regions):
    def freeze(a):
        return tuple(tuple(tuple(y) for y in x) for x in a)

    def step(st, r):
        pcs, cs, flags, data = st
        c, pc = cs[r], pcs[r]
        if c == calls:
            return None
        reg, epoch = c % regions, c + 1
        fl = [[list(y) for y in x] for x in flags]
        da = [[list(y) for y in x] for x in data]
        if pc < world:
            da[pc][reg][r] = c
        elif pc < 2 * world:
            p = pc - world
            assert fl[p][reg][r] < epoch, "epochs must grow"
            fl[p][reg][r] = epoch
        else:
            q = pc - 2 * world
            if flags[r][reg][q] < epoch:
                return None
            assert data[r][reg][q] == c, f"rank {r} call {c} read call {data[r][reg][q]} pushed by rank {q}"
        pc += 1
        pcs_l, cs_l = list(pcs), list(cs)
        if pc == 3 * world:
            pc, cs_l[r] = 0, c + 1
        pcs_l[r] = pc
        return (tuple(pcs_l), tuple(cs_l), freeze(fl), freeze(da))

    zeros = tuple(tuple(tuple([0] * world) for _ in range(regions)) for _ in range(world))
    minus = tuple(tuple(tuple([-1] * world) for _ in range(regions)) for _ in range(world))
    init = (tuple([0] * world), tuple([0] * world), zeros, minus)
    return init, step, (lambda st: all(c == calls for c in st[1])), (lambda st: None)


def test_allgather_two_regions_are_enough():
    for world, calls in ((2, 4), (3, 3)):
        init, step, done, final = _allgather_model(world, calls, regions=2)
        states, finals = _explore(init, step, done, final)
        assert states > 100 and finals >= 1


def test_allgather_one_region_is_caught():
    init, step, done, final = _allgather_model(2, 3, regions=1)
    try:
        _explore(init, step, done, final)
    except AssertionError:
        return
    raise AssertionError("the single-region protocol should have shown an overwritten row")
