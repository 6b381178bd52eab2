"""Random-schedule search of the attention kernels' mbarrier protocols on the host model
(tests/mbarrier_pipeline_model.py): no schedule may deadlock, overwrite a buffer that still has a
reader due, or read a buffer before it holds the expected step's data. The one protocol that is
KNOWN to be wrong (a two-slot statistics ring released by a once-per-step barrier) must be caught,
which shows the search has teeth."""
import pytest

import mbarrier_pipeline_model as M


@pytest.mark.parametrize("sep,qs", [(False, 3), (True, 3), (False, 2), (True, 4)])
def test_backward_pipelines_survive_random_schedules(sep, qs):
    """head_dim 64 (S^T / dP^T share columns) and head_dim 128 (separate columns) backward."""
    for steps in (1, 2, 3, 7, 12):
        for seed in range(40):
            M.backward_kv(seed, steps, qs=qs, sep=sep)
            M.backward_kv(seed, steps, qs=qs, sep=sep, producer_lag=400)   # and with a slow producer


@pytest.mark.parametrize("p_over_s,stages", [(False, 3), (False, 2), (True, 1), (True, 2)])
def test_forward_one_tile_pipelines_survive_random_schedules(p_over_s, stages):
    for steps in (1, 2, 3, 8, 17):
        for seed in range(40):
            M.forward_one_tile(seed, steps, stages=stages, p_over_s=p_over_s)


def test_the_search_finds_the_statistics_ring_that_deadlocked():
    """Statistics rows in a ring of their own, two slots, released through the once-per-step
    "dS stored" barrier: a producer that lags more than one step behind waits for a parity that
    has come round again. The model must find a schedule that shows it."""
    found = 0
    for seed in range(200):
        try:
            M.backward_kv(seed, 9, qs=3, sep=False, stats_with_stage=False, producer_lag=400)
        except (M.Deadlock, AssertionError):
            found += 1
    assert found > 0


def test_barrier_parity_is_the_hardware_test():
    b = M.Barrier("b", 2)
    assert b.passed(1) and not b.passed(0)          # fresh barrier: "previous" phase counts as done
    b.arrive(); assert not b.passed(0)
    b.arrive(); assert b.passed(0) and not b.passed(1)
    b.arrive(); b.arrive()
    assert b.passed(1) and not b.passed(0)          # two completions later the old parity blocks again


def test_gemm_epilogue_lookahead_never_overwrites_a_buffer_in_use():
    """The two staging sets of the fused FC2-dgrad epilogue: a set is reloaded only after the
    store that was sent from it has read it, whatever the delays of loads and stores."""
    for pieces in (1, 2, 3, 4, 9, 16):
        for seed in range(60):
            M.gemm_epilogue_lookahead(seed, pieces)


def test_cta_pair_gemm_protocol_survives_random_schedules():
    """The barrier protocol of the CTA-pair GEMM (not built: it stopped making progress next to
    other kernels on the GPU): no random schedule of loads, commits and remote arrivals deadlocks
    it, aliases a phase, reuses a stage or an accumulator too early, or lets an arrival reach a
    CTA that has exited. The search therefore does not explain the stall seen on the GPU, which
    supports looking for it in the instructions that no wait limit bounds."""
    for tiles, k_steps in ((1, 1), (1, 3), (2, 7), (3, 16), (5, 2)):
        for seed in range(40):
            M.pair_gemm(seed, tiles, k_steps)
            M.pair_gemm(seed, tiles, k_steps, stages=2)


def test_transaction_barrier_takes_bytes_before_the_expecting_arrival():
    b = M.TxBarrier("full", 1)
    b.complete_tx(1)                     # the partner's bytes land first
    assert b.completed == 0
    b.arrive_expect(2)
    assert b.completed == 0              # own bytes still due
    b.complete_tx(1)
    assert b.completed == 1 and b.passed(0)


@pytest.mark.parametrize("ks,vs", [(3, 3), (1, 1), (2, 1)])
def test_forward_two_tile_pipeline_survives_random_schedules(ks, vs):
    """Two query tiles sharing one K / V ring (a stage goes back after BOTH issuing warps have
    committed it); the first tile sees one block fewer than the second."""
    for blocks in (2, 3, 4, 9, 16):
        for seed in range(40):
            M.forward_two_tiles(seed, blocks, ks=ks, vs=vs)


def test_allgather_gemm_needs_the_whole_grid_resident():
    """The all-gather -> GEMM kernel's CTAs wait for chunks that other CTAs of the same grid copy:
    with every CTA resident the grid always drains; when fewer CTAs can run than the grid has, the
    resident ones end up waiting for a CTA that cannot start (on the GPU: the bounded wait runs
    out and reports a status). The host side therefore refuses a grid that the device cannot
    hold (``tp_grid_fits`` in csrc/gemm_tp_sm100.cu)."""
    for seed in range(20):
        M.allgather_gemm(seed, ctas=12, chunks=4, tiles=60, resident=12)
    stuck = 0
    for seed in range(20):
        try:
            M.allgather_gemm(seed, ctas=12, chunks=4, tiles=60, resident=5)
        except M.Deadlock:
            stuck += 1
    assert stuck == 20


@pytest.mark.parametrize("stages", [3, 4, 6])
def test_single_cta_gemm_pipeline_survives_random_schedules(stages):
    """Work items of different length (split-K pieces of 1 to 9 K steps, half tiles with fewer
    bytes per stage), odd and even stage counts (the two producers take stages by parity)."""
    import random
    for seed in range(40):
        rng = random.Random(seed)
        ks = [rng.randint(1, 9) for _ in range(rng.randint(1, 7))]
        halves = {t for t in range(len(ks)) if rng.random() < 0.3}
        M.gemm_single_cta(seed, ks, stages=stages, halves=halves)
    M.gemm_single_cta(0, [], stages=stages)                     # a CTA without work


def test_the_gemm_model_sees_what_the_producer_tail_is_for():
    """While barrier arrivals are delivered in the order of their commits, the epilogue's wait for
    the last accumulator covers every earlier stage release and the producers' closing waits are
    redundant. Once an arrival may lag behind a later one, a CTA without those waits can leave
    while a stage release is still on its way to its shared memory; with them it cannot. A release
    barrier that expects more epilogue arrivals than there are warps never opens."""
    for seed in range(40):
        M.gemm_single_cta(seed, [2, 3, 1], stages=4, producer_tail=False)
        M.gemm_single_cta(seed, [2, 3, 1], stages=4, producer_tail=True, arrival_skew=True)
    late = 0
    for seed in range(40):
        try:
            M.gemm_single_cta(seed, [2, 3, 1], stages=4, producer_tail=False, arrival_skew=True)
        except AssertionError as e:
            assert "after it had exited" in str(e) or "still in flight" in str(e)
            late += 1
    assert late > 0
    with pytest.raises(M.Deadlock):
        M.gemm_single_cta(0, [2, 2, 2, 2], stages=4, epi_threads=4, tempty_count=5)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_planes_are_never_overwritten_before_they_are_summed(world):
    for seed in range(25):
        M.gemm_reduce_scatter_stream(seed, world, launches=6)


def test_the_reduce_scatter_model_sees_why_there_are_two_plane_sets_a_barrier_and_a_fence():
    """One plane set: a fast peer's next launch overwrites a plane that the owner has not summed yet.
    No exit barrier: the owner sums a plane that has not arrived. A flag that overtakes the stores
    (no fence before the release): the same. Each is found within a few seeds."""
    def fails(**kw):
        n = 0
        for seed in range(40):
            try:
                M.gemm_reduce_scatter_stream(seed, 4, launches=6, **kw)
            except AssertionError:
                n += 1
        return n
    assert fails(planes=1) > 0
    assert fails(exit_barrier=False) > 0
    assert fails(fenced=False) > 0
    assert fails() == 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gathered_slots_are_rewritten_only_after_every_peer_has_read_them(world):
    for seed in range(25):
        M.allgather_gemm_stream(seed, world, launches=6)
    broken = 0
    for seed in range(40):
        try:
            M.allgather_gemm_stream(seed, world, launches=6, exit_barrier=False)
        except AssertionError:
            broken += 1
    assert broken > 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_parameter_buckets_are_replaced_only_between_a_steps_last_read_and_the_next_first_read(world):
    for seed in range(20):
        M.dp_param_pipeline(seed, world, steps=4)


def test_the_parameter_pipeline_model_sees_what_the_norm_all_reduce_and_the_exit_barrier_are_for():
    """Without the all-reduce of the gradient norm a fast rank pushes new parameters into a peer that
    is still reading the old ones; without the exit barrier a rank's next forward reads a bucket
    into which a peer's shard has not been pushed yet."""
    def fails(**kw):
        n = 0
        for seed in range(40):
            try:
                M.dp_param_pipeline(seed, 4, steps=4, **kw)
            except AssertionError:
                n += 1
        return n
    assert fails(norm_allreduce=False) > 0
    assert fails(exit_barrier=False) > 0
    assert fails() == 0
