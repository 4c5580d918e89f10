"""Event-driven CPU model of the mbarrier protocol of the prefill kernel (csrc/varlen_prefill.cu).

The kernel's five roles -- TMA producer, two MMA issuers, two softmax warpgroups -- only meet through mbarriers whose
waits see one parity bit.  The model replays their exact sequence of waits / arrivals / tcgen05.commit for random item
lists under randomised latencies and checks what the hardware cannot tell us without a hang:

  * no deadlock (every role runs to the end of the item list);
  * no parity alias: when a wait for phase k passes, exactly k+1 phases have completed (a barrier that got two phases
    ahead of an observer would either release it early or block it forever);
  * no barrier receives more arrivals than its count within a phase;
  * a K/V ring slot is never refilled before both issuers have released it;
  * the softmax warpgroup that zeroes the rows past a sequence's end in its last V tile waits for that slot only
    at such tiles (skipping every other phase of the slot), and still never sees another tile there.

The tensor pipe is modelled as an in-order queue (a commit arrives when everything its thread issued before has
finished), TMA loads as delayed arrivals.
"""
import heapq
import random

import pytest

SLOTS = 5  # K/V ring slots, filled K0 V0 K1 V1 ...


class ProtocolError(Exception):
    pass


class Bar:
    def __init__(self, name, count):
        self.name, self.count, self.pending, self.completed, self.waiters = name, count, count, 0, []


class Sim:
    def __init__(self, seed, jitter):
        self.t, self.q, self.n, self.rng, self.jitter = 0.0, [], 0, random.Random(seed), jitter
        self.threads, self.pipe_free = {}, 0.0

    def lat(self, x):
        return x * (1 + self.jitter * (2 * self.rng.random() - 1)) + self.jitter * 300 * self.rng.random()

    def at(self, t, fn):
        self.n += 1
        heapq.heappush(self.q, (t, self.n, fn))

    def spawn(self, name, gen):
        self.threads[name] = gen
        self.at(0.0, lambda: self.step(name))

    def arrive(self, bar):
        bar.pending -= 1
        if bar.pending < 0:
            raise ProtocolError(f"{bar.name}: more arrivals than its count")
        if bar.pending == 0:
            bar.pending, bar.completed = bar.count, bar.completed + 1
            waiters, bar.waiters = bar.waiters, []
            for name, phase in waiters:
                self.wait(name, bar, phase)

    def wait(self, name, bar, phase):
        if (bar.completed & 1) != (phase & 1):  # what mbarrier.try_wait.parity sees
            if bar.completed != phase + 1:
                raise ProtocolError(f"{name}: wait for phase {phase} of {bar.name} passed at {bar.completed} completions")
            self.at(self.t + self.lat(150), lambda: self.step(name))
        else:
            if bar.completed > phase + 1:
                raise ProtocolError(f"{name}: {bar.name} ran ahead of phase {phase} ({bar.completed}): would never pass")
            bar.waiters.append((name, phase))

    def step(self, name):
        try:
            cmd = next(self.threads[name])
        except StopIteration:
            del self.threads[name]
            return
        if cmd[0] == "wait":
            self.wait(name, cmd[1], cmd[2])
        elif cmd[0] == "arrive":
            self.arrive(cmd[1])
            self.at(self.t, lambda: self.step(name))
        elif cmd[0] == "delay":
            self.at(self.t + self.lat(cmd[1]), lambda: self.step(name))
        elif cmd[0] == "tma":  # asynchronous completion on the barrier
            self.at(self.t + self.lat(1800), lambda b=cmd[1]: self.arrive(b))
            self.at(self.t + 20, lambda: self.step(name))
        elif cmd[0] == "mma":  # in-order tensor pipe; commits arrive when the batch (and all before it) is done
            end = max(self.t, self.pipe_free) + cmd[1]
            self.pipe_free = end
            for b in cmd[2]:
                self.at(end + self.lat(60), lambda b=b: self.arrive(b))
            self.at(max(self.t + 20, end - 128), lambda: self.step(name))
        else:
            raise ValueError(cmd)

    def run(self):
        while self.q:
            self.t, _, fn = heapq.heappop(self.q)
            fn()
        if self.threads:
            raise ProtocolError(f"deadlock: {sorted(self.threads)} never finished")


def run_cta(items, seed=0, jitter=0.0, empty_count=2, hand_turn_back=True):
    """items: per work item (n_a, n_b[, ragged]) = K/V tiles Q tile A / B visit (n_b = 0: no second tile) and whether
    the last V tile reaches past the sequence's end (the softmax warpgroups that use it zero those rows first)."""
    items = [it if len(it) == 3 else (it[0], it[1], False) for it in items]
    sim = Sim(seed, jitter)
    q_full, q_empty = Bar("q_full", 1), Bar("q_empty", 2)
    kv_full = [Bar(f"kv_full{s}", 1) for s in range(SLOTS)]
    kv_empty = [Bar(f"kv_empty{s}", empty_count) for s in range(SLOTS)]
    s_full = [Bar(f"s_full{x}", 1) for x in range(2)]
    p_full = [[Bar(f"p_full{x}{h}", 1) for h in range(2)] for x in range(2)]  # one arrival stands for the 4 warps
    o_full = [Bar(f"o_full{x}", 1) for x in range(2)]
    o_empty = [Bar(f"o_empty{x}", 1) for x in range(2)]
    turn = [Bar(f"turn{x}", 1) for x in range(2)]
    slot_tile = [None] * SLOTS  # ring position whose tile the slot holds (or is being filled with)
    slot_state = ["empty"] * SLOTS  # ring-slot invariant: empty -> loading -> full -> (both released) -> empty
    released = [0] * SLOTS

    def producer():
        kt = 0
        for i, (n_a, n_b, _) in enumerate(items):
            if i > 0:
                yield ("wait", q_empty, i - 1)
            yield ("tma", q_full)
            for _ in range(max(n_a, n_b)):
                for kv in range(2):
                    pos = 2 * kt + kv
                    s = pos % SLOTS
                    if pos >= SLOTS:
                        yield ("wait", kv_empty[s], pos // SLOTS - 1)
                    if slot_state[s] != "empty":
                        raise ProtocolError(f"slot {s} refilled while {slot_state[s]}")
                    slot_state[s] = "full"  # (readable once kv_full completes; reads are checked against the barrier)
                    slot_tile[s] = pos
                    yield ("tma", kv_full[s])
                kt += 1

    def release(s):
        released[s] += 1
        if released[s] == 2:
            released[s], slot_state[s] = 0, "empty"

    def issuer(x):
        kt = tiles = used = 0

        def slot(pos):
            return ("wait", kv_full[pos % SLOTS], pos // SLOTS)

        for i, (n_a, n_b, _) in enumerate(items):
            n_x, n_kv = (n_a, n_b)[x], max(n_a, n_b)
            yield ("wait", q_full, i)
            if n_x == 0:
                yield ("arrive", q_empty)
            kpos = 2 * kt
            yield slot(kpos)
            if n_x > 0:
                yield ("mma", 512, [s_full[x], kv_empty[kpos % SLOTS]] + ([q_empty] if n_x == 1 else []))
            else:
                yield ("arrive", kv_empty[kpos % SLOTS])
            release(kpos % SLOTS)
            for j in range(n_kv):
                vpos, kpos = 2 * (kt + j) + 1, 2 * (kt + j) + 2
                yield slot(vpos)
                if j + 1 < n_kv:  # K(j+1) is awaited before P.V(j) so that nothing is polled between the two MMA groups
                    yield slot(kpos)
                if j < n_x:
                    if j == 0 and used > 0:
                        yield ("wait", o_empty[x], used - 1)
                    yield ("wait", p_full[x][0], tiles)
                    yield ("mma", 256, [])
                    yield ("wait", p_full[x][1], tiles)
                    # the commits of P.V(j) follow the Q.K^T(j+1) MMAs when there are any
                    yield ("mma", 256, [] if j + 1 < n_x else [o_full[x], kv_empty[vpos % SLOTS]])
                    tiles += 1
                else:
                    yield ("arrive", kv_empty[vpos % SLOTS])
                if j + 1 < n_kv:
                    if j + 1 < n_x:
                        yield ("mma", 512, [s_full[x], kv_empty[kpos % SLOTS], o_full[x], kv_empty[vpos % SLOTS]]
                               + ([q_empty] if j + 2 == n_x else []))
                    else:
                        yield ("arrive", kv_empty[kpos % SLOTS])
                    release(kpos % SLOTS)
                release(vpos % SLOTS)
            used += 1 if n_x > 0 else 0
            kt += n_kv

    def softmax(x):
        tiles = turns_seen = kt = 0
        for n_a, n_b, ragged in items:
            n_x, n_kv = (n_a, n_b)[x], max(n_a, n_b)
            kt0, kt = kt, kt + n_kv
            both = n_b > 0
            for j in range(n_x):
                yield ("wait", s_full[x], tiles)
                if ragged and j == n_kv - 1:  # zero the rows past the sequence's end in V(last) before P is handed over
                    vpos = 2 * (kt0 + n_kv - 1) + 1
                    yield ("wait", kv_full[vpos % SLOTS], vpos // SLOTS)
                    if slot_tile[vpos % SLOTS] != vpos:
                        raise ProtocolError(f"softmax{x} zeroes rows of ring position {slot_tile[vpos % SLOTS]}, not {vpos}")
                    yield ("delay", 60)
                yield ("delay", 300)  # scores to registers, row max: not exclusive
                if both and (j >= 1 if x == 0 else j < n_a):  # A(j) after B(j-1); B(j) after A(j) while A has tiles
                    yield ("wait", turn[x ^ 1], turns_seen)
                    turns_seen += 1
                yield ("delay", 800)
                yield ("arrive", p_full[x][0])
                yield ("delay", 600)
                if both and (x == 0 or j + 1 < n_a) and (hand_turn_back or x == 0):
                    yield ("arrive", turn[x])  # handed over once the last chunk of P is on its way
                yield ("arrive", p_full[x][1])
                tiles += 1
            if n_x > 0:
                yield ("wait", o_full[x], tiles - 1)
                yield ("delay", 900)
                yield ("arrive", o_empty[x])

    sim.spawn("producer", producer())
    for x in range(2):
        sim.spawn(f"issuer{x}", issuer(x))
        sim.spawn(f"softmax{x}", softmax(x))
    sim.run()
    return sim.t


def item_tiles(q0, rows, prefix=0, last=None, pair_heads=False):
    """What load_item computes for the row block starting at row q0 with `rows` live rows of a sequence with
    `prefix` cached tokens; `last` says whether it is the sequence's final block (default: iff the block is not full).
    pair_heads: the item is 128 rows of two heads (both Q tiles see the same keys) instead of 256 rows of one head."""
    full = 128 if pair_heads else 256
    rows = min(rows, full)
    last = rows < full if last is None else last
    len_k = prefix + q0 + rows if last else prefix + q0 + rows + 300
    nk_total = -(-len_k // 128)
    n_a = min(nk_total, (prefix + q0 + 127) // 128 + 1)
    if pair_heads:
        n_b = n_a
    else:
        n_b = min(nk_total, (prefix + q0 + 255) // 128 + 1) if rows > 128 else 0
    return n_a, n_b, max(n_a, n_b) * 128 > len_k


def test_single_items_of_every_shape():
    for q0 in (0, 256, 1024):
        for rows in (1, 128, 129, 256):
            assert run_cta([item_tiles(q0, rows)]) > 0
            assert run_cta([item_tiles(q0, rows, pair_heads=True)]) > 0


@pytest.mark.parametrize("seed", range(40))
def test_random_item_lists_under_random_latencies(seed):
    rng = random.Random(seed)
    pair_heads = seed % 2 == 1
    items = [item_tiles((128 if pair_heads else 256) * rng.randint(0, 7), rng.choice([1, 64, 128, 129, 200, 256, 256, 256]),
                        prefix=rng.choice([0, 0, 1, 127, 128, 300]), last=rng.choice([None, None, True]),
                        pair_heads=pair_heads)
             for _ in range(rng.randint(1, 14))]
    for jitter in (0.0, 0.4, 0.95):
        run_cta(items, seed=seed, jitter=jitter)


def test_model_catches_broken_protocols():
    """The checker itself must report protocols that are wrong on purpose."""
    items = [item_tiles(512, 256)] * 3
    with pytest.raises(ProtocolError):  # a ring slot released by one issuer only: refilled while the other reads it
        run_cta(items, empty_count=1)
    with pytest.raises(ProtocolError, match="deadlock"):  # tile B never hands the softmax turn back
        run_cta(items, hand_turn_back=False)
