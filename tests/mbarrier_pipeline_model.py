"""Host model of the mbarrier pipelines of the tensor-core kernels (attention:
csrc/attn_bwd_kv_sm100.cu, csrc/attn_bwd_kv128_sm100.cu, csrc/attn_fwd1_sm100.cu,
csrc/attn_fwd_sm100.cu; GEMM: csrc/gemm_sm100.cu; tensor-parallel GEMM + collective:
csrc/gemm_tp_sm100.cu): which role waits on which barrier with which parity, who arrives, and
which resources (TMEM columns, shared-memory buffers, peer-memory planes) a barrier or flag
guards. The model exists to search the protocols for two classes of design errors without a GPU:

* deadlock, including the "phase aliasing" kind: an mbarrier only knows the parity of its current
  phase, so a waiter that is still waiting for completion k when completion k+2 has happened blocks
  for good. ``Barrier.passed`` is the hardware's test: ``try_wait.parity(p)`` succeeds iff the
  number of completed phases is odd when p == 0 and even when p == 1.
* a resource written while its previous content is still to be read (write-after-read), or read
  before it was written: every buffer carries the step number of its content and the number of
  readers still due.

Roles are Python generators that yield requests; a scheduler picks a runnable role at random and
delivers asynchronous completions (TMA loads, tensor-core commits) after random delays. Commits of
one issuing thread complete in issue order, like the tensor pipe's."""
from __future__ import annotations

import random


class Barrier:
    def __init__(self, name: str, count: int):
        self.name, self.count = name, count
        self.pending = count
        self.completed = 0          # phases completed so far

    def arrive(self, n: int = 1) -> None:
        self.pending -= n
        assert self.pending >= 0, f"{self.name}: more arrivals than its count in one phase"
        if self.pending == 0:
            self.completed += 1
            self.pending = self.count

    def passed(self, parity: int) -> bool:
        return (self.completed & 1) != (parity & 1)


class Resource:
    """A buffer or a group of TMEM columns: content tag + readers still due."""

    def __init__(self, name: str):
        self.name = name
        self.tag = None
        self.readers_due = 0

    def write(self, tag, readers: int) -> None:
        assert self.readers_due == 0, \
            f"{self.name}: overwritten with {tag} while {self.readers_due} reader(s) of {self.tag} are due"
        self.tag, self.readers_due = tag, readers

    def read(self, tag) -> None:
        assert self.tag == tag, f"{self.name}: holds {self.tag}, reader expected {tag}"
        assert self.readers_due > 0, f"{self.name}: more reads of {tag} than announced"
        self.readers_due -= 1


class Deadlock(AssertionError):
    pass


class Sim:
    """Roles yield ``("wait", barrier, parity)``, ``("wait_fn", predicate, name)``, ``("arrive",
    barrier)``, ``("async", delay_rank, fn)`` (fn runs later; asyncs of one ``delay_rank`` keep
    their order) or ``("step",)``."""

    def __init__(self, seed: int):
        self.rng = random.Random(seed)
        self.roles: list[tuple[str, object]] = []
        self.blocked: dict[int, tuple[Barrier, int]] = {}
        self.queues: dict[object, list] = {}     # per issuing engine: FIFO of pending completions
        self.now = 0
        self.slow_prefix: str | None = None      # queues of this name prefix deliver reluctantly

    def add(self, name: str, gen) -> None:
        self.roles.append((name, gen))

    @staticmethod
    def _free(entry) -> bool:
        what, arg = entry
        return what.passed(arg) if isinstance(what, Barrier) else what()

    @staticmethod
    def _describe(entry):
        what, arg = entry
        return (what.name, arg, what.completed) if isinstance(what, Barrier) else arg

    def run(self, limit: int = 2_000_000) -> None:
        alive = set(range(len(self.roles)))
        for _ in range(limit):
            self.now += 1
            # deliver the head of a random engine queue now and then
            live_q = [k for k, q in self.queues.items() if q]
            if self.slow_prefix is not None:      # an adversarial schedule: these come as late as possible
                live_q = [k for k in live_q if not (isinstance(k, str) and k.startswith(self.slow_prefix)
                                                    and self.rng.random() < 0.95)]
            if live_q and self.rng.random() < 0.35:
                k = self.rng.choice(live_q)
                self.queues[k].pop(0)()
            runnable = [i for i in alive if i not in self.blocked or self._free(self.blocked[i])]
            if not runnable:
                live_q = [k for k, q in self.queues.items() if q]
                if live_q:
                    k = self.rng.choice(live_q)
                    self.queues[k].pop(0)()
                    continue
                if not alive:
                    return
                waits = {self.roles[i][0]: self._describe(self.blocked[i]) for i in alive}
                raise Deadlock(f"no role can run: {waits}")
            i = self.rng.choice(runnable)
            self.blocked.pop(i, None)
            try:
                req = next(self.roles[i][1])
            except StopIteration:
                alive.discard(i)
                continue
            if req[0] == "wait":
                if not req[1].passed(req[2]):
                    self.blocked[i] = (req[1], req[2])
            elif req[0] == "wait_fn":
                if not req[1]():
                    self.blocked[i] = (req[1], req[2])
            elif req[0] == "arrive":
                req[1].arrive()
            elif req[0] == "async":
                self.queues.setdefault(req[1], []).append(req[2])
        raise AssertionError("simulation did not finish")


# ---------------------------------------------------------------------------------------------
# attention backward, TMEM-operand kernels. ``sep`` = S^T and dP^T in separate TMEM columns (the
# head_dim 128 kernel); else they share columns and dP^T is issued when S^T is in registers.
# ---------------------------------------------------------------------------------------------
def backward_kv(seed: int, steps: int, qs: int = 3, sep: bool = False, softmax_threads: int = 4,
                drain_threads: int = 2, stats_with_stage: bool = True, producer_lag: int = 0) -> None:
    sim = Sim(seed)
    ns, nd = softmax_threads, drain_threads
    B = lambda n, c=1: Barrier(n, c)
    kv_full = B("kv_full")
    qdo_full = [B(f"qdo_full{s}") for s in range(qs)]
    qdo_empty = [B(f"qdo_empty{s}") for s in range(qs)]
    s_full, s_free = B("s_full"), B("s_free", ns)
    dp_full, dp_free = B("dp_full"), B("dp_free", ns)
    p_ready, p_free = B("p_ready", ns), B("p_free")
    pds_ready, dst_free, ds_free = B("pds_ready", ns), B("dst_free"), B("ds_free")
    dq_full, dq_drained, dkv_full = B("dq_full"), B("dq_drained", nd), B("dkv_full")
    # one-phase statistics ring of two slots released by pds_ready (the design that deadlocked)
    stat_full = [B(f"stat_full{s}") for s in range(2)]
    stage = [Resource(f"stage{s}") for s in range(qs)]
    stat = [Resource(f"stat{s}") for s in range(2)]
    S, dP = Resource("S^T"), Resource("dP^T")
    SdP = Resource("S^T/dP^T")
    Pt, dSt, dSs, dQ = Resource("P^T"), Resource("dS^T tmem"), Resource("dS^T smem"), Resource("dQ")
    N = steps

    def producer():
        yield ("async", "tma", kv_full.arrive)
        for n in range(N):
            s = n % qs
            for _ in range(int(sim.rng.random() * producer_lag)):   # a producer that falls behind
                yield ("step",)
            yield ("wait", qdo_empty[s], ((n // qs) & 1) ^ 1)
            readers = 4 + (ns if stats_with_stage else 0)     # S, dP, dV, dK (+ statistics)
            def landed(s=s, n=n, readers=readers):
                stage[s].write(("qdo", n), readers)
                qdo_full[s].arrive()
            yield ("async", "tma", landed)
            if not stats_with_stage:
                t = n % 2
                # this ring's release is the once-per-step pds_ready of step n-2
                if n >= 2:
                    yield ("wait", pds_ready, (n - 2) & 1)
                def stat_landed(t=t, n=n):
                    stat[t].write(("stat", n), ns)
                    stat_full[t].arrive()
                yield ("async", "tma2", stat_landed)

    def mma():
        def issue(reads, write, done_bars):
            def fn():
                for r, tag in reads:
                    r.read(tag)
                if write is not None:
                    write[0].write(write[1], write[2])
                for b in done_bars:
                    b.arrive()
            return ("async", "tensor", fn)
        yield ("wait", kv_full, 0)
        yield ("wait", qdo_full[0], 0)
        Sres = S if sep else SdP
        dPres = dP if sep else SdP
        yield issue([(stage[0], ("qdo", 0))], (Sres, ("S", 0), ns), [s_full])
        if sep:
            yield issue([(stage[0], ("qdo", 0))], (dPres, ("dP", 0), ns), [dp_full])
        for n in range(N):
            st = stage[n % qs]
            if not sep:
                yield ("wait", s_free, n & 1)
                yield issue([(st, ("qdo", n))], (dPres, ("dP", n), ns), [dp_full])
            yield ("wait", p_ready, n & 1)
            yield issue([(Pt, ("P", n)), (st, ("qdo", n))], None, [p_free])            # dV
            if n + 1 < N:
                nx = stage[(n + 1) % qs]
                if sep:
                    yield ("wait", s_free, n & 1)
                    yield ("wait", qdo_full[(n + 1) % qs], ((n + 1) // qs) & 1)
                    yield issue([(nx, ("qdo", n + 1))], (Sres, ("S", n + 1), ns), [s_full])
                    yield ("wait", dp_free, n & 1)
                    yield issue([(nx, ("qdo", n + 1))], (dPres, ("dP", n + 1), ns), [dp_full])
                else:
                    yield ("wait", dp_free, n & 1)
                    yield ("wait", qdo_full[(n + 1) % qs], ((n + 1) // qs) & 1)
                    yield issue([(nx, ("qdo", n + 1))], (Sres, ("S", n + 1), ns), [s_full])
            yield ("wait", pds_ready, n & 1)
            yield issue([(dSt, ("dS", n)), (st, ("qdo", n))], None,
                        [dst_free, qdo_empty[n % qs]])                                   # dK
            if n > 0:
                yield ("wait", dq_drained, (n - 1) & 1)
            yield issue([(dSs, ("dS", n))], (dQ, ("dQ", n), nd), [dq_full, ds_free])      # dQ
        yield ("async", "tensor", dkv_full.arrive)

    def softmax(lag: float):
        Sres = S if sep else SdP
        dPres = dP if sep else SdP
        for n in range(N):
            for _ in range(int(sim.rng.random() * lag)):
                yield ("step",)
            s = n % qs
            yield ("wait", qdo_full[s], (n // qs) & 1)
            if stats_with_stage:
                stage[s].read(("qdo", n))          # the statistics rows of the stage
            else:
                yield ("wait", stat_full[n % 2], (n // 2) & 1)
                stat[n % 2].read(("stat", n))
            yield ("wait", s_full, n & 1)
            Sres.read(("S", n))
            yield ("arrive", s_free)
            if n > 0:
                yield ("wait", p_free, (n - 1) & 1)
            Pt.write(("P", n), 1) if Pt.tag != ("P", n) else None
            yield ("arrive", p_ready)
            yield ("wait", dp_full, n & 1)
            dPres.read(("dP", n))
            yield ("arrive", dp_free)
            if n > 0:
                yield ("wait", dst_free, (n - 1) & 1)
                yield ("wait", ds_free, (n - 1) & 1)
            if dSt.tag != ("dS", n):
                dSt.write(("dS", n), 1)
                dSs.write(("dS", n), 1)
            yield ("arrive", pds_ready)

    def drain():
        for n in range(N):
            yield ("wait", dq_full, n & 1)
            dQ.read(("dQ", n))
            yield ("arrive", dq_drained)
        yield ("wait", dkv_full, 0)

    sim.add("producer", producer())
    sim.add("mma", mma())
    for i in range(ns):
        sim.add(f"softmax{i}", softmax(lag=0 if i else 6))
    for i in range(nd):
        sim.add(f"drain{i}", drain())
    sim.run()


# ---------------------------------------------------------------------------------------------
# attention forward, one query tile per CTA. ``p_over_s``: the probabilities are written over
# the score columns and the next score block is issued behind the P V product (head_dim 128).
# ---------------------------------------------------------------------------------------------
def forward_one_tile(seed: int, steps: int, stages: int = 3, p_over_s: bool = False,
                     softmax_threads: int = 4) -> None:
    sim = Sim(seed)
    ns = softmax_threads
    B = lambda n, c=1: Barrier(n, c)
    q_full = B("q_full")
    k_full = [B(f"k_full{s}") for s in range(stages)]
    k_empty = [B(f"k_empty{s}") for s in range(stages)]
    v_full = [B(f"v_full{s}") for s in range(stages)]
    v_empty = [B(f"v_empty{s}") for s in range(stages)]
    s_full, s_free, p_ready, o_done = B("s_full"), B("s_free", ns), B("p_ready", ns), B("o_done")
    K = [Resource(f"K{s}") for s in range(stages)]
    V = [Resource(f"V{s}") for s in range(stages)]
    S, P = Resource("S"), Resource("P")
    N = steps

    def producer(which, full, empty, bufs):
        if which == "k":
            yield ("async", "tma_q", q_full.arrive)
        for j in range(N):
            s = j % stages
            yield ("wait", empty[s], ((j // stages) & 1) ^ 1)
            def landed(s=s, j=j):
                bufs[s].write((which, j), 1)
                full[s].arrive()
            yield ("async", "tma_" + which, landed)

    def mma():
        def issue_S(j):
            def fn():
                K[j % stages].read(("k", j))
                if p_over_s and j > 0:
                    assert P.readers_due == 0, "score block issued over probabilities still to be read"
                S.write(("S", j), ns)
                s_full.arrive()
                k_empty[j % stages].arrive()
            return ("async", "tensor", fn)
        def issue_PV(j):
            def fn():
                P.read(("P", j))
                V[j % stages].read(("v", j))
                o_done.arrive()
                v_empty[j % stages].arrive()
            return ("async", "tensor", fn)
        yield ("wait", q_full, 0)
        yield ("wait", k_full[0], 0)
        yield issue_S(0)
        for j in range(N):
            if not p_over_s and j + 1 < N:
                yield ("wait", s_free, j & 1)
                yield ("wait", k_full[(j + 1) % stages], ((j + 1) // stages) & 1)
                yield issue_S(j + 1)
            yield ("wait", v_full[j % stages], (j // stages) & 1)
            yield ("wait", p_ready, j & 1)
            yield issue_PV(j)
            if p_over_s and j + 1 < N:
                yield ("wait", k_full[(j + 1) % stages], ((j + 1) // stages) & 1)
                yield issue_S(j + 1)

    def softmax(lag: float):
        for j in range(N):
            for _ in range(int(sim.rng.random() * lag)):
                yield ("step",)
            yield ("wait", s_full, j & 1)
            S.read(("S", j))
            if not p_over_s:
                yield ("arrive", s_free)
            if j > 0:
                yield ("wait", o_done, (j - 1) & 1)
            if P.tag != ("P", j):
                P.write(("P", j), 1)
            yield ("arrive", p_ready)
        yield ("wait", o_done, (N - 1) & 1)

    sim.add("producer_k", producer("k", k_full, k_empty, K))
    sim.add("producer_v", producer("v", v_full, v_empty, V))
    sim.add("mma", mma())
    for i in range(ns):
        sim.add(f"softmax{i}", softmax(lag=0 if i else 6))
    sim.run()


# ---------------------------------------------------------------------------------------------
# GEMM with the SwiGLU backward in the epilogue: one epilogue warp's two staging sets. For piece i
# the gate / up boxes land in set i % 2 (TMA load, barrier yb[set]), the warp reads them, writes
# the results back into the same set and sends them off (TMA store, bulk group); the loads of
# piece i+1 are issued during piece i, after the stores of piece i-1 have read set (i+1) % 2.
# ---------------------------------------------------------------------------------------------
def gemm_epilogue_lookahead(seed: int, pieces: int, tiles_every: int = 4) -> None:
    sim = Sim(seed)
    yb = [Barrier("yb0", 1), Barrier("yb1", 1)]
    tfull = [Barrier("tfull0", 1), Barrier("tfull1", 1)]      # two TMEM accumulators
    tempty = [Barrier("tempty0", 1), Barrier("tempty1", 1)]
    sets = [Resource("set0"), Resource("set1")]
    stores_in_flight: list[int] = []     # bulk groups committed and not yet read, oldest first
    n_tiles = (pieces + tiles_every - 1) // tiles_every

    def mma():   # fills accumulator t % 2 once the epilogue has released it
        for t in range(n_tiles):
            yield ("wait", tempty[t % 2], ((t >> 1) & 1) ^ 1)
            yield ("async", "tensor", tfull[t % 2].arrive)

    def issue_load(i):
        s = i % 2
        def landed():
            sets[s].write(("in", i), 1)
            yb[s].arrive()
        return ("async", "tma_load", landed)

    def warp():
        if pieces:
            yield issue_load(0)      # the first piece's boxes: before the first accumulator is awaited
        for i in range(pieces):
            s = i % 2
            t = i // tiles_every
            if i % tiles_every == 0:
                yield ("wait", tfull[t % 2], (t >> 1) & 1)
            yield ("wait", yb[s], (i >> 1) & 1)
            sets[s].read(("in", i))
            if i + 1 < pieces:
                # wait_group_read<0>: every committed store has read its buffer
                while stores_in_flight:
                    yield ("step",)
                yield issue_load(i + 1)
            sets[s].write(("out", i), 1)
            def store_read(s=s, i=i):
                sets[s].read(("out", i))
                stores_in_flight.remove(i)
            stores_in_flight.append(i)
            yield ("async", "tma_store", store_read)
            if i % tiles_every == tiles_every - 1 or i == pieces - 1:
                yield ("arrive", tempty[t % 2])
        while stores_in_flight:
            yield ("step",)

    sim.add("mma", mma())
    sim.add("warp", warp())
    sim.run()


# ---------------------------------------------------------------------------------------------
# CTA-pair GEMM (the kernel that is not built, csrc/gemm_sm100.cu behind FT_BUILD_PAIR_GEMM): two
# CTAs, each with its own operand ring; the leader issues every product and its commits arrive at
# the same-named barrier of BOTH CTAs; both CTAs' loads report to the LEADER's full barrier (one
# arrival with the expected byte count from the leader's producer, bytes from both); the epilogue
# threads of both CTAs release an accumulator on the leader's barrier. A CTA must not exit while
# an arrival addressed to it is still on its way.
# ---------------------------------------------------------------------------------------------
class TxBarrier(Barrier):
    """mbarrier with a transaction count: a phase completes when the pending arrivals AND the
    outstanding bytes are both zero (bytes may be reported before the arrival that expects them)."""

    def __init__(self, name: str, count: int):
        super().__init__(name, count)
        self.tx = 0

    def _check(self) -> None:
        if self.pending == 0 and self.tx == 0:
            self.completed += 1
            self.pending = self.count

    def arrive(self, n: int = 1) -> None:
        self.pending -= n
        assert self.pending >= 0, f"{self.name}: more arrivals than its count in one phase"
        self._check()

    def arrive_expect(self, nbytes: int) -> None:
        self.tx += nbytes
        self.arrive()

    def complete_tx(self, nbytes: int) -> None:
        self.tx -= nbytes
        self._check()


def pair_gemm(seed: int, tiles: int, k_steps: int, stages: int = 6, epi_threads: int = 2) -> None:
    sim = Sim(seed)
    E = epi_threads
    full = [TxBarrier(f"full{s}", 1) for s in range(stages)]                       # leader only
    empty = [[Barrier(f"empty{c}_{s}", 1) for s in range(stages)] for c in range(2)]
    tfull = [[Barrier(f"tfull{c}_{b}", 1) for b in range(2)] for c in range(2)]
    tempty = [Barrier(f"tempty{b}", 2 * E) for b in range(2)]                      # leader only
    bufs = [[Resource(f"stage{c}_{s}") for s in range(stages)] for c in range(2)]
    acc = [[Resource(f"acc{c}_{b}") for b in range(2)] for c in range(2)]
    exited = [False, False]
    done = [0, 0]            # roles of a CTA that have finished
    roles_per_cta = [1 + 1 + E, 1 + E]

    def to_cta(c, fn):
        def deliver():
            assert not exited[c], f"an arrival reached CTA {c} after it had exited"
            fn()
        return deliver

    def producer(c):
        use = 0
        for _t in range(tiles):
            for _k in range(k_steps):
                s = use % stages
                yield ("wait", empty[c][s], ((use // stages) & 1) ^ 1)
                if c == 0:
                    full[s].arrive_expect(2)       # one unit of bytes per CTA
                def landed(c=c, s=s, use=use):
                    bufs[c][s].write(("ops", use), 1)
                    full[s].complete_tx(1)
                yield ("async", f"tma{c}", to_cta(0, landed))
                use += 1
        # tail: observe the release of every stage once more
        for _ in range(stages):
            s = use % stages
            yield ("wait", empty[c][s], ((use // stages) & 1) ^ 1)
            use += 1
        done[c] += 1

    def mma():
        use = 0
        for t in range(tiles):
            b = t & 1
            yield ("wait", tempty[b], ((t >> 1) & 1) ^ 1)
            for _k in range(k_steps):
                s = use % stages
                yield ("wait", full[s], (use // stages) & 1)
                def ran(s=s, use=use, b=b, t=t, first=(_k == 0)):
                    for c in range(2):
                        bufs[c][s].read(("ops", use))
                        if first:
                            acc[c][b].write(("acc", t), E)
                def released(s=s):
                    pass
                yield ("async", "tensor", ran)
                for c in range(2):     # one commit, delivered to both CTAs' barriers
                    yield ("async", "tensor", to_cta(c, empty[c][s].arrive))
                use += 1
            for c in range(2):
                yield ("async", "tensor", to_cta(c, tfull[c][b].arrive))
        for t in range(tiles, tiles + 2):      # tail: both accumulators released by everybody
            yield ("wait", tempty[t & 1], ((t >> 1) & 1) ^ 1)
        done[0] += 1

    def epilogue(c):
        for t in range(tiles):
            b = t & 1
            yield ("wait", tfull[c][b], (t >> 1) & 1)
            acc[c][b].read(("acc", t))
            yield ("async", f"remote{c}", to_cta(0, tempty[b].arrive))
        done[c] += 1

    def cta_exit(c):
        # __syncthreads, cluster barrier, free, cluster barrier: modelled as "both CTAs' roles done"
        while done[0] < roles_per_cta[0] or done[1] < roles_per_cta[1]:
            yield ("step",)
        exited[c] = True

    sim.add("producer0", producer(0))
    sim.add("producer1", producer(1))
    sim.add("mma", mma())
    for c in range(2):
        for i in range(E):
            sim.add(f"epilogue{c}_{i}", epilogue(c))
        sim.add(f"exit{c}", cta_exit(c))
    sim.run()
    # nothing may still be on its way once both CTAs are gone
    assert not any(sim.queues.values()), "arrivals still in flight after both CTAs exited"


# ---------------------------------------------------------------------------------------------
# attention forward, two query tiles per CTA (csrc/attn_fwd_sm100.cu): one K / V ring shared by
# two issuing warps (a stage returns to the producer after BOTH have committed it), tile 0 sees
# one score block fewer than tile 1 on the causal diagonal.
# ---------------------------------------------------------------------------------------------
def forward_two_tiles(seed: int, blocks: int, ks: int = 3, vs: int = 3, softmax_threads: int = 2,
                      p_single_buffer_wait_first: bool = False) -> None:
    sim = Sim(seed)
    ns = softmax_threads
    B = lambda n, c=1: Barrier(n, c)
    q_full = B("q_full")
    k_full = [B(f"k_full{s}") for s in range(ks)]
    k_empty = [B(f"k_empty{s}", 2) for s in range(ks)]
    v_full = [B(f"v_full{s}") for s in range(vs)]
    v_empty = [B(f"v_empty{s}", 2) for s in range(vs)]
    s_full = [B(f"s_full{w}") for w in range(2)]
    s_free = [B(f"s_free{w}", ns) for w in range(2)]
    p_ready = [B(f"p_ready{w}", ns) for w in range(2)]
    o_done = [B(f"o_done{w}") for w in range(2)]
    K = [Resource(f"K{s}") for s in range(ks)]
    V = [Resource(f"V{s}") for s in range(vs)]
    S = [Resource(f"S{w}") for w in range(2)]
    P = [Resource(f"P{w}") for w in range(2)]
    n_total = blocks
    nk = [blocks - 1, blocks]          # tile 0 skips the last block

    def producer(which, full, empty, bufs, depth):
        if which == "k":
            yield ("async", "tma_q", q_full.arrive)
        for j in range(n_total):
            s = j % depth
            yield ("wait", empty[s], ((j // depth) & 1) ^ 1)
            readers = 2 if j < nk[0] else 1
            def landed(s=s, j=j, readers=readers):
                bufs[s].write((which, j), readers)
                full[s].arrive()
            yield ("async", "tma_" + which, landed)

    def mma(w):
        def issue_S(j):
            def fn():
                K[j % ks].read(("k", j))
                S[w].write(("S", j), ns)
                s_full[w].arrive()
                k_empty[j % ks].arrive()
            return ("async", "tensor", fn)
        def issue_PV(j):
            def fn():
                P[w].read(("P", j))
                V[j % vs].read(("v", j))
                o_done[w].arrive()
                v_empty[j % vs].arrive()
            return ("async", "tensor", fn)
        if nk[w] == 0:
            return
        yield ("wait", q_full, 0)
        yield ("wait", k_full[0], 0)
        yield issue_S(0)
        for j in range(nk[w]):
            if j + 1 < nk[w]:
                yield ("wait", s_free[w], j & 1)
                yield ("wait", k_full[(j + 1) % ks], ((j + 1) // ks) & 1)
                yield issue_S(j + 1)
            yield ("wait", v_full[j % vs], (j // vs) & 1)
            yield ("wait", p_ready[w], j & 1)
            yield issue_PV(j)
        # (tile 0 never touches the last block and does not return that stage: it is the last
        # load of the CTA, nobody waits for the stage again)

    def softmax(w, lag):
        for j in range(nk[w]):
            for _ in range(int(sim.rng.random() * lag)):
                yield ("step",)
            yield ("wait", s_full[w], j & 1)
            S[w].read(("S", j))
            yield ("arrive", s_free[w])
            if j > 0:
                yield ("wait", o_done[w], (j - 1) & 1)
            if P[w].tag != ("P", j):
                P[w].write(("P", j), 1)
            yield ("arrive", p_ready[w])
        if nk[w]:
            yield ("wait", o_done[w], (nk[w] - 1) & 1)

    sim.add("producer_k", producer("k", k_full, k_empty, K, ks))
    sim.add("producer_v", producer("v", v_full, v_empty, V, vs))
    for w in range(2):
        sim.add(f"mma{w}", mma(w))
        for i in range(ns):
            sim.add(f"softmax{w}_{i}", softmax(w, lag=0 if i else 5))
    sim.run()


# ---------------------------------------------------------------------------------------------
# all-gather -> GEMM (csrc/gemm_tp_sm100.cu, mode 1): every CTA's copy warps bring one part of
# one remote 128-row chunk into local memory and bump that chunk's counter; a CTA's TMA producer
# may load a remote row block once its counter has reached the number of parts. CTAs therefore
# wait for one another: the grid has to be resident as a whole. ``resident`` limits how many CTAs
# run at a time (a CTA takes a slot when one is free and keeps it until it ends).
# ---------------------------------------------------------------------------------------------
def allgather_gemm(seed: int, ctas: int, chunks: int, tiles: int, resident: int) -> None:
    sim = Sim(seed)
    group = max(1, ctas // chunks)               # CTAs that share one chunk
    ready = [0] * chunks
    state = {"finished": 0}

    def cta(i):
        # CTAs are launched in order as SMs have room: CTA i starts once i - resident + 1 have ended
        yield ("wait_fn", lambda: state["finished"] >= i - resident + 1, f"launch of CTA {i}")
        # copy warps: this CTA's part of "its" chunk (at most one chunk per CTA, as in the kernel)
        c = i // group
        if c < chunks:
            yield ("step",)
            ready[c] += 1
        # producer: tiles i, i + ctas, ...; local row blocks need no chunk, remote ones wait for theirs
        for t in range(i, tiles, ctas):
            need = t % (chunks + 1)              # 0: a local row block
            if need:
                yield ("wait_fn", lambda need=need: ready[need - 1] >= group, f"chunk {need - 1}")
            yield ("step",)
        state["finished"] += 1

    for i in range(ctas):
        sim.add(f"cta{i}", cta(i))
    sim.run()


# ---------------------------------------------------------------------------------------------
# single-CTA GEMM (csrc/gemm_sm100.cu, gemm_bf16_kernel): two producer warps that take the
# stages of their own parity, one issuing warp, epilogue warps that drain one of two TMEM
# accumulators. Work items have different numbers of K steps (split-K pieces) and byte counts
# (half tiles load half of the B boxes). A barrier arrival of the tensor pipe must not reach the
# CTA after it has exited, which is what the producers' tail waits are for.
# ---------------------------------------------------------------------------------------------
def gemm_single_cta(seed: int, k_steps: list[int], stages: int = 4, epi_threads: int = 4,
                    halves: set[int] = frozenset(), producer_tail: bool = True,
                    tempty_count: int | None = None, arrival_skew: bool = False) -> None:
    """``arrival_skew``: commits still complete in issue order, but the arrival that a commit sends
    to a stage barrier is delivered after a delay of its own, as late as the schedule allows (it may
    be overtaken by the arrival of a later commit at an accumulator barrier)."""
    sim = Sim(seed)
    sim.slow_prefix = "late_"
    E = epi_threads
    full = [TxBarrier(f"full{s}", 1) for s in range(stages)]
    empty = [Barrier(f"empty{s}", 1) for s in range(stages)]
    tfull = [Barrier(f"tfull{b}", 1) for b in range(2)]
    tempty = [Barrier(f"tempty{b}", tempty_count or E) for b in range(2)]
    bufs = [Resource(f"stage{s}") for s in range(stages)]
    acc = [Resource(f"acc{b}") for b in range(2)]
    state = {"done": 0, "exited": False}
    n_roles = 2 + 1 + E

    def guarded(bar):
        def deliver():
            assert not state["exited"], "a tensor-pipe arrival reached the CTA after it had exited"
            bar.arrive()
        if not arrival_skew or not bar.name.startswith("empty"):
            return deliver
        return lambda: sim.queues.setdefault(f"late_{bar.name}", []).append(deliver)

    def producer(pid):
        use = 0
        for t, kn in enumerate(k_steps):
            boxes = 2 if t in halves else 3          # A + half of B, or A + both B boxes
            for _k in range(kn):
                s = use % stages
                if (s & 1) == pid:
                    yield ("wait", empty[s], ((use // stages) & 1) ^ 1)
                    full[s].arrive_expect(boxes)
                    bufs[s].write(("ops", use), 1)   # the stage is the producer's from here on
                    for j in range(boxes):           # one box per lane, each its own copy
                        yield ("async", f"tma{pid}_{j}", lambda s=s: full[s].complete_tx(1))
                use += 1
        if producer_tail:
            for _ in range(stages):
                s = use % stages
                if (s & 1) == pid:
                    yield ("wait", empty[s], ((use // stages) & 1) ^ 1)
                use += 1
        state["done"] += 1

    def mma():
        use = 0
        for t, kn in enumerate(k_steps):
            b = t & 1
            yield ("wait", tempty[b], ((t >> 1) & 1) ^ 1)
            for k in range(kn):
                s = use % stages
                yield ("wait", full[s], (use // stages) & 1)

                def ran(s=s, use=use, b=b, t=t, first=(k == 0)):
                    bufs[s].read(("ops", use))
                    if first:
                        acc[b].write(("acc", t), E)
                yield ("async", "tensor", ran)
                yield ("async", "tensor", guarded(empty[s]))
                use += 1
            yield ("async", "tensor", guarded(tfull[b]))
        state["done"] += 1

    def epilogue():
        for t in range(len(k_steps)):
            b = t & 1
            yield ("wait", tfull[b], (t >> 1) & 1)
            acc[b].read(("acc", t))
            yield ("arrive", tempty[b])
        state["done"] += 1

    def cta_exit():
        yield ("wait_fn", lambda: state["done"] >= n_roles, "every role of the CTA")
        state["exited"] = True

    sim.add("producer0", producer(0))
    sim.add("producer1", producer(1))
    sim.add("mma", mma())
    for i in range(E):
        sim.add(f"epilogue{i}", epilogue())
    sim.add("exit", cta_exit())
    sim.run()
    assert not any(sim.queues.values()), "arrivals still in flight after the CTA exited"


# ---------------------------------------------------------------------------------------------
# Streams of tensor-parallel launches over several ranks (csrc/gemm_tp_sm100.cu with
# parallel/fused_tp.py). A rank is one role: its launches run one after the other, like kernels
# of one stream. Stores into a peer's memory land later, in issue order per source rank (the
# kernel fences them before it releases its flag); a flag release travels on the same queue when
# ``fenced`` and overtakes the stores otherwise.
# ---------------------------------------------------------------------------------------------
def gemm_reduce_scatter_stream(seed: int, world: int, launches: int, planes: int = 2,
                               exit_barrier: bool = True, fenced: bool = True) -> None:
    """GEMM -> reduce-scatter: rank r stores its partial tiles into plane r of every owner (the
    plane set alternates between ``planes`` halves), the ranks meet in the exit barrier, and each
    owner's next kernel sums its planes."""
    sim = Sim(seed)
    plane = [[[Resource(f"plane[{o}][{h}][{s}]") for s in range(world)] for h in range(planes)]
             for o in range(world)]
    flag = [[0] * world for _ in range(world)]        # flag[dst][src]: last epoch signalled

    def rank(r):
        for n in range(1, launches + 1):
            h = n % planes
            for o in range(world):                    # remote owners first, as the kernel does
                o = (r + 1 + o) % world
                yield ("async", f"stores{r}", lambda o=o, h=h, n=n: plane[o][h][r].write(n, 1))
            if exit_barrier:
                for d in range(world):
                    if d != r:
                        def signal(d=d, n=n):
                            flag[d][r] = n
                        yield ("async", f"stores{r}" if fenced else f"flags{r}", signal)
                for s in range(world):
                    if s != r:
                        yield ("wait_fn", lambda s=s, n=n: flag[r][s] >= n, f"rank {r}: exit flag of {s}")
                # own stores: complete when the kernel ends (bulk-store wait before the barrier)
                yield ("wait_fn", lambda: not sim.queues.get(f"stores{r}"), f"rank {r}: own stores")
            yield ("step",)
            for s in range(world):                    # the sum kernel that follows on the stream
                plane[r][h][s].read(n)
                yield ("step",)

    for r in range(world):
        sim.add(f"rank{r}", rank(r))
    sim.run()


def allgather_gemm_stream(seed: int, world: int, launches: int, exit_barrier: bool = True) -> None:
    """All-gather -> GEMM: before launch n every rank has written its own slot; the kernel tells the
    peers so, pulls their slots once they have said the same, and leaves through the exit barrier
    ("I no longer read your slot"), after which the stream's next producer may overwrite the slot."""
    sim = Sim(seed)
    slot = [Resource(f"slot{r}") for r in range(world)]
    ready = [[0] * world for _ in range(world)]       # ready[dst][src]
    done = [[0] * world for _ in range(world)]

    def rank(r):
        for n in range(1, launches + 1):
            slot[r].write(n, world - 1)               # the producer kernel before the launch
            yield ("step",)
            for d in range(world):
                if d != r:
                    ready[d][r] = n
            for s in range(world):
                s = (r + 1 + s) % world
                if s == r:
                    continue
                yield ("wait_fn", lambda s=s, n=n: ready[r][s] >= n, f"rank {r}: slot of {s}")
                yield ("step",)
                slot[s].read(n)
            if exit_barrier:
                for d in range(world):
                    if d != r:
                        done[d][r] = n
                for s in range(world):
                    if s != r:
                        yield ("wait_fn", lambda s=s, n=n: done[r][s] >= n, f"rank {r}: exit flag of {s}")
            yield ("step",)

    for r in range(world):
        sim.add(f"rank{r}", rank(r))
    sim.run()


# ---------------------------------------------------------------------------------------------
# Data-parallel step over several ranks (trainer.py, optim/adamw.py, parallel/fused_dp.py,
# csrc/comm.cu): forward and backward read the parameter buckets; the squared gradient norm is
# all-reduced (every rank passes it after its last read of the old parameters); then, bucket by
# bucket in forward-consumption order on a side stream, the fused AdamW kernel pushes this rank's
# updated shard into EVERY rank's parameter buffer and leaves through an exit barrier; the next
# forward waits for a bucket's event right before the first layer that reads it.
# ---------------------------------------------------------------------------------------------
def dp_param_pipeline(seed: int, world: int, steps: int, n_buckets: int = 3,
                      norm_allreduce: bool = True, exit_barrier: bool = True) -> None:
    sim = Sim(seed)
    # shard[r][b][s]: rank r's copy of bucket b, the shard owned by rank s
    shard = [[[Resource(f"params[{r}][{b}][{s}]") for s in range(world)] for b in range(n_buckets)]
             for r in range(world)]
    for r in range(world):
        for b in range(n_buckets):
            for s in range(world):
                shard[r][b][s].write(0, 2)            # version 0, read by forward and backward of step 1
    norm_seen = [[0] * world for _ in range(world)]   # norm_seen[dst][src]: last step signalled
    done = [[[0] * world for _ in range(world)] for _ in range(n_buckets)]    # exit flags per bucket
    gathered = [[0] * n_buckets for _ in range(world)]                        # event per bucket

    def main_stream(r):
        for n in range(1, steps + 1):
            for b in reversed(range(n_buckets)):      # forward: embedding's bucket (last) first
                yield ("wait_fn", lambda b=b, n=n: gathered[r][b] >= n - 1, f"rank {r}: bucket {b} of step {n - 1}")
                for s in range(world):
                    shard[r][b][s].read(n - 1)
                yield ("step",)
            for b in range(n_buckets):                # backward: data gradients read the weights
                for s in range(world):
                    shard[r][b][s].read(n - 1)
                yield ("step",)
            if norm_allreduce:
                for d in range(world):
                    norm_seen[d][r] = n
                for s in range(world):
                    yield ("wait_fn", lambda s=s, n=n: norm_seen[r][s] >= n, f"rank {r}: norm of {s}")
            # hand the step over to the side stream (an event in the engine)
            handed[r] = n
            yield ("step",)

    handed = [0] * world

    def side_stream(r):
        for n in range(1, steps + 1):
            yield ("wait_fn", lambda n=n: handed[r] >= n, f"rank {r}: gradients of step {n}")
            for b in reversed(range(n_buckets)):
                for d in range(world):                # update + push of the own shard to every rank
                    yield ("async", f"push{r}", lambda d=d, b=b, n=n: shard[d][b][r].write(n, 2))
                if exit_barrier:
                    for d in range(world):
                        def signal(d=d, b=b, n=n):
                            done[b][d][r] = n
                        yield ("async", f"push{r}", signal)       # released after the stores (fence)
                    for s in range(world):
                        yield ("wait_fn", lambda s=s, b=b, n=n: done[b][r][s] >= n,
                               f"rank {r}: exit flag of {s} for bucket {b}")
                else:
                    yield ("wait_fn", lambda: not sim.queues.get(f"push{r}"), f"rank {r}: own pushes")
                gathered[r][b] = n
                yield ("step",)

    for r in range(world):
        sim.add(f"main{r}", main_stream(r))
        sim.add(f"side{r}", side_stream(r))
    sim.run()
