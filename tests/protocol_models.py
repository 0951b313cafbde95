"""Event-driven models of the block-level protocols of the single-launch backward kernels.

They model WHO WAITS FOR WHAT and WHO PUBLISHES WHAT, exactly as the kernels do it
(flexsae_b200/csrc/flexsae_backward.cuh: decoder_loss_bwd_pipelined_kernel;
flexsae_b200/csrc/flexsae_sharded.cuh: decoder_loss_bwd_sharded_kernel;
flexsae_b200/csrc/flexsae_small_allreduce.cuh: small_allreduce_kernel), with blocks dispatched in
index order into a limited number of resident slots and random durations, and check the protocol
itself: no circular wait whatever the number of resident blocks (down to one), nothing read before
it is complete, nothing overwritten before it has been read, every conversion exactly once.  They
say nothing about the CUDA code beyond that; the GPU tests do.  Test infrastructure only.
"""
import heapq
import random


class Hazard(AssertionError):
    pass


def run_sharded(R, P, U, E, C, exch_off, conv_off, in_place, slots, seed, steps=2, ordered=True, ns=2, lag=1):
    """R ranks, P pieces, per slot U unit / E exchange / C converting blocks; `ns` slabs in rotation and
    the scatter of a piece `lag` slots behind its accumulation (1 <= lag < ns); `in_place`: reduced rows
    go straight into the peers' dweight (exchange waits for scatter flags only); `ordered`: a rank's
    flags are published strictly in slot order (what the kernel does; False shows what that rule prevents)."""
    L = lag
    rnd = random.Random(seed)
    speed = [rnd.uniform(0.5, 2.0) for _ in range(R)]
    nslots = P + L + 2
    last_slot, last_scatter_slot = P + L + 1, P + L - 1
    flagsE = [[0]*R for _ in range(R)]; flagsC = [[0]*R for _ in range(R)]   # [at rank][of rank]
    inbox = [[[(-1, 0, -1) for _ in range(R)] for _ in range(2)] for _ in range(R)]     # [owner][parity][sender] = (piece, writes, step)
    reduced = {}   # (step, owner, piece) -> number of exch blocks that reduced it
    gathered = [[[(-1, 0, -1) for _ in range(R)] for _ in range(2)] for _ in range(R)]  # [dest][parity][owner]
    copied = {}    # (step, dest, piece) -> exch blocks that copied
    landed = {}    # (step, dest, piece, owner) -> blocks that wrote dW rows in place
    t = 0.0; heap = []; waiting = []; seq = [0]
    errors = []
    def exch_count(p): return E if p < P + L else E + C      # blocks that share the exchange work of slot p
    def make_rank(r, step_no):
        seq_base = 1 + step_no * (P + 5)      # what flexsae_shard_slots answers: an upper bound of the slots
        walk_done = [0]*(nslots); conv_done = [0]*nslots; slot_done = [0]*nslots; scat_done = [0]*nslots
        slab = [(-1, "free")] * ns             # (piece, "accumulating" | "free"): what each slab holds
        def publish(kind, p):
            for s in range(R):
                (flagsC if kind == "C" else flagsE)[s][r] = seq_base + p
        def waitE(target): return lambda: all(flagsE[r][s] >= target for s in range(R))
        def waitC(target): return lambda: all(flagsC[r][s] >= target for s in range(R))
        def unit(p):
            if p >= ns: yield ("wait", lambda: conv_done[p - ns + L] >= C)
            held = slab[p % ns]
            if held[1] != "free" and held[0] != p: errors.append(("walk started on an unconverted slab", r, p, held))
            slab[p % ns] = (p, "accumulating")
            yield ("work", rnd.uniform(5, 30) * speed[r])
            walk_done[p] += 1
        def conv(p):
            q = p - L
            if 0 <= q < P:
                yield ("wait", lambda: walk_done[q] >= U)
                yield ("wait", waitE(seq_base + p - 1))
                if slab[q % ns][0] != q: errors.append(("converted a slab that holds another piece", r, q, slab[q % ns]))
                yield ("work", rnd.uniform(1, 6) * speed[r])
                for o in range(R):
                    pc, wr, st = inbox[o][q & 1][r]
                    if (pc, st) != (q, step_no):
                        # first writer of this piece: previous content must have been reduced completely
                        if pc >= 0 and reduced.get((st, o, pc), 0) < exch_count(pc + L + 1):
                            errors.append(("inbox overwritten before reduce", r, o, q, pc, st))
                        inbox[o][q & 1][r] = (q, 1, step_no)
                    else:
                        inbox[o][q & 1][r] = (q, wr + 1, step_no)
            conv_done[p] += 1
            if 0 <= q < P and conv_done[p] == C: slab[q % ns] = (q, "free")
            scat_done[p] += 1
            if scat_done[p] == C:
                if ordered and p > 0: yield ("wait", lambda: flagsC[r][r] >= seq_base + p - 1)
                publish("C", p)
        def exch(p):
            n = exch_count(p)
            if p >= 2:
                if (not in_place) or p == last_slot: yield ("wait", waitE(seq_base + p - 1))
                yield ("wait", waitC(seq_base + min(p - 1, last_scatter_slot)))
            q = p - L - 1
            if 0 <= q < P:
                for s in range(R):
                    if inbox[r][q & 1][s] != (q, C, step_no): errors.append(("reduce reads incomplete inbox", r, s, q, inbox[r][q & 1][s]))
                yield ("work", rnd.uniform(1, 6) * speed[r])
                for s in range(R):
                    if inbox[r][q & 1][s] != (q, C, step_no): errors.append(("inbox changed during reduce", r, s, q, inbox[r][q & 1][s]))
                reduced[(step_no, r, q)] = reduced.get((step_no, r, q), 0) + 1
                for o in range(R):
                    if o == r: continue
                    if in_place:
                        landed[(step_no, o, q, r)] = landed.get((step_no, o, q, r), 0) + 1
                    else:
                        pc, wr, st = gathered[o][q & 1][r]
                        if (pc, st) != (q, step_no):
                            if pc >= 0 and copied.get((st, o, pc), 0) < exch_count(pc + L + 2):
                                errors.append(("gather buffer overwritten before copy", r, o, q, pc))
                            gathered[o][q & 1][r] = (q, 1, step_no)
                        else:
                            gathered[o][q & 1][r] = (q, wr + 1, step_no)
            q = p - L - 2
            if 0 <= q < P and not in_place:
                for ow in range(R):
                    if ow != r and gathered[r][q & 1][ow] != (q, exch_count(q + L + 1), step_no):
                        errors.append(("copy reads incomplete gather buffer", r, ow, q, gathered[r][q & 1][ow]))
                yield ("work", rnd.uniform(0.5, 3) * speed[r])
                copied[(step_no, r, q)] = copied.get((step_no, r, q), 0) + 1
            slot_done[p] += 1
            if slot_done[p] == n:
                if ordered and p > 0: yield ("wait", lambda: flagsE[r][r] >= seq_base + p - 1)
                publish("E", p)
        order = []
        for p in range(P):
            row = []
            for i in range(U + C):
                if i >= conv_off and i < conv_off + C: row.append(("conv", p))
                else: row.append(("unit", p))
            row = row[:exch_off] + [("exch", p)] * E + row[exch_off:]   # exch_off <= conv_off
            order += row
        for d in range(L + 2):
            p = P + d
            order += ([("exch", p)] * E + [("conv", p)] * C) if d < L else [("exch", p)] * (E + C)
        gens = {"unit": unit, "conv": conv, "exch": exch}
        return [gens[k](p) for k, p in order]
    # each rank runs `steps` kernels back to back (stream order): next kernel's blocks start after the previous finished
    state = []
    for r in range(R):
        state.append({"step": 0, "blocks": make_rank(r, 0), "nxt": 0, "active": 0, "done": 0})
    def step_gen(r, g):
        st = state[r]
        try:
            kind, arg = next(g)
        except StopIteration:
            st["active"] -= 1; st["done"] += 1
            return
        if kind == "work":
            seq[0] += 1; heapq.heappush(heap, (t + arg, seq[0], r, g))
        else:
            waiting.append((arg, r, g))
    def fill(r):
        st = state[r]
        while True:
            if st["nxt"] >= len(st["blocks"]):
                if st["done"] == len(st["blocks"]) and st["step"] + 1 < steps:
                    # in place: every peer's rows of every piece must have landed before the kernel ended
                    if in_place:
                        for q in range(P):
                            for ow in range(R):
                                if ow != r and landed.get((st["step"], r, q, ow), 0) < E:
                                    errors.append(("kernel ended before all rows landed", r, q, ow))
                    st["step"] += 1; st["blocks"] = make_rank(r, st["step"]); st["nxt"] = 0; st["done"] = 0
                    continue
                return
            if st["active"] >= slots: return
            g = st["blocks"][st["nxt"]]; st["nxt"] += 1; st["active"] += 1
            step_gen(r, g)
    for r in range(R): fill(r)
    guard = 0
    def all_done(): return all(s["step"] == steps - 1 and s["done"] == len(s["blocks"]) for s in state)
    while not all_done():
        guard += 1; assert guard < 5 * 10**6
        progressed = True
        while progressed:
            progressed = False
            for item in list(waiting):
                cond, r, g = item
                if cond():
                    waiting.remove(item); step_gen(r, g); progressed = True
            for r in range(R): fill(r)
        if all_done(): break
        if not heap:
            raise Hazard(f"deadlock: {len(waiting)} blocks waiting")
        t, _, r, g = heapq.heappop(heap)
        step_gen(r, g)
        for rr in range(R): fill(rr)
    if in_place:
        for r in range(R):
            for q in range(P):
                for ow in range(R):
                    if ow != r and landed.get((steps - 1, r, q, ow), 0) < E: errors.append(("last kernel: rows missing", r, q, ow))
    if errors:
        raise Hazard(str(errors[:5]))


def run_pipelined(P, U, C, conv_off, slots, seed, ns=2, lag=1):
    """decoder_loss_bwd_pipelined_kernel: slot p holds the U unit blocks of piece p with the C blocks that
    convert piece p - lag inserted at `conv_off`; `lag` trailing slots of C converting blocks; `ns` slabs in
    rotation.  Unit blocks of piece p wait for the conversion of piece p - ns (same slab), converting
    blocks for the walk of their piece."""
    rnd = random.Random(seed)
    walk_done = [0] * P
    conv_done = [0] * P
    problems = []
    slab = [(-1, "free")] * ns

    def unit(p):
        if p >= ns:
            yield ("wait", lambda: conv_done[p - ns] >= C)
        if slab[p % ns][1] != "free" and slab[p % ns][0] != p:
            problems.append(("walk started on an unconverted slab", p, slab[p % ns]))
        slab[p % ns] = (p, "accumulating")
        yield ("work", rnd.uniform(5, 40))
        walk_done[p] += 1

    def conv(q):
        if q < 0:
            return
        yield ("wait", lambda: walk_done[q] >= U)
        if slab[q % ns][0] != q:
            problems.append(("converted a slab that holds another piece", q, slab[q % ns]))
        yield ("work", rnd.uniform(1, 6))
        conv_done[q] += 1
        if conv_done[q] == C:
            slab[q % ns] = (q, "free")

    order = []
    for p in range(P):
        row = [("unit", p)] * U
        row = row[:conv_off] + [("conv", p - lag)] * C + row[conv_off:]
        order += row
    for d in range(lag):
        order += [("conv", P + d - lag)] * C
    blocks = [(unit if k == "unit" else conv)(i) for k, i in order]
    t, heap, waiting, seq, nxt, active, done = 0.0, [], [], 0, 0, 0, 0

    def advance(g):
        nonlocal seq, active, done
        try:
            kind, arg = next(g)
        except StopIteration:
            active -= 1
            done += 1
            return
        if kind == "work":
            seq += 1
            heapq.heappush(heap, (t + arg, seq, g))
        else:
            waiting.append((arg, g))

    def fill():
        nonlocal nxt, active
        while active < slots and nxt < len(blocks):
            g = blocks[nxt]
            nxt += 1
            active += 1
            advance(g)

    fill()
    while done < len(blocks):
        moved = True
        while moved:
            moved = False
            for item in list(waiting):
                if item[0]():
                    waiting.remove(item)
                    advance(item[1])
                    moved = True
            fill()
        if done >= len(blocks):
            break
        if not heap:
            raise Hazard(f"deadlock: {len(waiting)} blocks waiting, {done} of {len(blocks)} finished")
        t, _, g = heapq.heappop(heap)
        advance(g)
        fill()
    if any(c != C for c in conv_done) or any(w != U for w in walk_done):
        problems.append((walk_done, conv_done))
    if problems:
        raise Hazard(str(problems))
    return t


def run_small_allreduce(R, calls, seed):
    """small_allreduce_kernel: call number n (1, 2, ...) of rank r stores its value into cell [n & 1][r]
    of every rank, announces n in every rank's flag array, waits until every sender has announced n
    and reads the cells.  Calls of one rank run one after the other (stream order).  Checked: every
    read sees the value of the same call number (two cells per sender are enough)."""
    rnd = random.Random(seed)
    cells = [[[0] * R for _ in range(2)] for _ in range(R)]      # [at rank][parity][sender] = call number stored
    flags = [[0] * R for _ in range(R)]                          # [at rank][sender]
    events = []                                                  # (time, seq, rank, phase, call)
    seq = 0
    for r in range(R):
        heapq.heappush(events, (rnd.uniform(0, 5), seq, r, "push", 1))
        seq += 1
    waiting = []
    finished = [0] * R
    t = 0.0
    while events or waiting:
        if not events:
            raise Hazard(f"deadlock: {len(waiting)} ranks waiting")
        t, _, r, phase, n = heapq.heappop(events)
        if phase == "push":
            for o in range(R):
                cells[o][n & 1][r] = n
            for o in range(R):
                flags[o][r] = n
            waiting.append((r, n))
        elif phase == "read":
            for s_ in range(R):
                if cells[r][n & 1][s_] != n:
                    raise Hazard(f"rank {r} call {n} read sender {s_}'s cell holding call {cells[r][n & 1][s_]}")
            finished[r] = n
            if n < calls:
                seq += 1
                heapq.heappush(events, (t + rnd.uniform(0, 5), seq, r, "push", n + 1))
        for item in list(waiting):
            rr, nn = item
            if all(flags[rr][s_] >= nn for s_ in range(R)):
                waiting.remove(item)
                seq += 1
                heapq.heappush(events, (t + rnd.uniform(0, 3), seq, rr, "read", nn))    # the read takes a while
    if any(f != calls for f in finished):
        raise Hazard(str(finished))
