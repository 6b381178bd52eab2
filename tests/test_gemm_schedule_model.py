"""Index arithmetic of the GEMM kernels, checked on the CPU over many shapes (the model is
``gemm_schedule_model.py``): coverage of the output by work units, K pieces, half tiles of the last
wave, TMA box coordinates, and the tile order of the tensor-parallel kernels."""
import random

import pytest

import gemm_schedule_model as S

# shapes the engine launches: (name, M, N, K) of the 0.5B model at 16384 tokens and of one TP=2
# rank of the 8B model at 4096 / 8192 tokens, forward / dgrad / wgrad orientation
MODEL_SHAPES = [
    ("0.5b qkv", 16384, 1280, 1024), ("0.5b attn_out", 16384, 1024, 1024), ("0.5b fc1", 16384, 8192, 1024),
    ("0.5b fc2", 16384, 1024, 4096), ("0.5b head", 16384, 73448, 1024),
    ("0.5b qkv dgrad", 16384, 1024, 1280), ("0.5b fc1 dgrad", 16384, 1024, 8192),
    ("0.5b qkv wgrad", 1280, 1024, 16384), ("0.5b fc1 wgrad", 8192, 1024, 16384),
    ("0.5b fc2 wgrad", 1024, 4096, 16384), ("0.5b head wgrad", 73448, 1024, 16384),
    ("8b qkv", 4096, 2304, 4096), ("8b attn_out", 4096, 4096, 2048), ("8b fc1", 4096, 16384, 4096),
    ("8b fc2", 4096, 4096, 8192), ("8b head", 4096, 36728, 4096), ("8b fc2 wgrad", 4096, 8192, 8192),
]


def test_the_sources_still_say_what_the_model_restates():
    gemm = (S.CSRC / "gemm_sm100.cu").read_text()
    for line in ("if (rem > 0 && 2 * rem <= max_ctas) {", "kb = ks * base + min(ks, rem);",
                 "kn = base + (ks < rem ? 1 : 0);", "if (splitk > 16) splitk = 16;",
                 "const int max_by_k = k_iters / 8 > 0 ? k_iters / 8 : 1;",
                 "if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;",
                 "mt = first_m + in % gm;", "nt = in / gm;"):
        assert line in gemm, line
    tp = (S.CSRC / "gemm_tp_sm100.cu").read_text()
    for line in ("if (grid >= 2 && rem > 0 && 2 * rem <= grid) {", "mt = (ml + rot) % p.m_tiles;",
                 "const int rot = p.mode == 1 ? p.rank * p.tiles_per_slot"):
        assert line in tp, line
    assert S.G == {"GEMM_BM": 128, "GEMM_BK": 64, "GEMM_GROUP_M": 16}
    assert S.T["TP_BM"] == 128 and S.T["TP_BN"] == 256 and S.T["TP_MAX"] == 8


def _check_coverage(p: S.Plan):
    """Every output tile gets every K step exactly once; half tiles come in pairs that split the
    tile's columns; no unit has an empty K range."""
    seen: dict[tuple[int, int, int], list[tuple[int, int]]] = {}
    for u in range(p.total_units):
        mt, nt, kb, kn, half = S.decode_tile(p, u)
        assert 0 <= mt < p.m_tiles and 0 <= nt < p.n_tiles
        assert kn >= 1 and 0 <= kb and kb + kn <= p.k_iters
        if half >= 0:
            assert p.splitk == 1 and u >= p.split_from and p.bn == 256
        for h in ((0, 1) if half < 0 else (half,)):
            seen.setdefault((mt, nt, h), []).append((kb, kn))
    assert len(seen) == 2 * p.m_tiles * p.n_tiles
    for key, pieces in seen.items():
        pieces.sort()
        assert pieces[0][0] == 0 and pieces[-1][0] + pieces[-1][1] == p.k_iters, key
        assert all(a[0] + a[1] == b[0] for a, b in zip(pieces, pieces[1:])), key
        assert len(pieces) == p.splitk


@pytest.mark.parametrize("name,M,N,K", MODEL_SHAPES)
def test_model_shapes_are_covered_once_in_every_orientation(name, M, N, K):
    for out_f32, acc in ((False, False), (True, False), (True, True)):
        p = S.plan_gemm(M, N, K, out_f32=out_f32, accumulate=acc)
        _check_coverage(p)
        # several K pieces write the same output: they must add, and a plain store must not be split
        assert (p.splitk > 1) <= (p.out_mode == "f32_add")
        assert p.out_mode == ("bf16" if not out_f32 else p.out_mode)


def test_random_shapes_grids_and_forced_parameters_are_covered_once():
    rng = random.Random(1)
    for _ in range(400):
        M, N, K = rng.randint(1, 3000), rng.randint(1, 3000), rng.randint(1, 5000)
        kw = dict(out_f32=rng.random() < 0.5, max_ctas=rng.choice([0, 1, 2, 3, 37, 148, 500]),
                  bn=rng.choice([0, 128, 256]), splitk=rng.choice([0, 0, 1, 2, 5, 64]))
        kw["accumulate"] = kw["out_f32"] and rng.random() < 0.5
        p = S.plan_gemm(M, N, K, **kw)
        _check_coverage(p)
        assert 1 <= p.grid <= 148 and p.grid <= p.total_units
        assert p.splitk <= p.k_iters
        if not kw["out_f32"]:
            assert p.splitk == 1


def test_tail_split_only_cuts_a_last_wave_that_is_at_most_half_full():
    for name, M, N, K in MODEL_SHAPES:
        p = S.plan_gemm(M, N, K)
        total = p.m_tiles * p.n_tiles
        rem = total % 148
        if p.split_from < total:
            assert 0 < rem <= 74 and p.total_units == total + rem and p.split_from == total - rem
            # after the cut the last wave is full or the units divide evenly over the CTAs' turns
            assert (p.total_units - (total - rem)) == 2 * rem <= 148
        else:
            assert rem == 0 or rem > 74 or p.bn != 256
    # the shapes named in the kernel's comment
    assert S.plan_gemm(16384, 1024, 1024).total_units == 512 + 68
    assert S.plan_gemm(16384, 1280, 1024).total_units == 640 + 48
    assert S.plan_gemm(16384, 8192, 1024).total_units == 4096       # 27.7 waves: not cut


def test_weight_gradients_with_few_tiles_split_the_token_dimension():
    p = S.plan_gemm(1024, 1024, 16384, out_f32=True)                 # attn_out wgrad: 32 tiles
    assert p.splitk == 4 and p.total_units == 128 and p.out_mode == "f32_add"
    p = S.plan_gemm(1280, 1024, 16384, out_f32=True)                 # qkv wgrad: 40 tiles
    assert p.splitk == 3 and p.total_units == 120
    p = S.plan_gemm(1024, 1024, 256, out_f32=True)                   # too little K to split
    assert p.splitk == 1 and p.out_mode == "f32"
    p = S.plan_gemm(128, 128, 1 << 20, out_f32=True)                 # one tile: capped at 16 ways
    assert p.splitk == 16
    _check_coverage(p)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_every_tma_box_starts_on_a_16_byte_boundary_inside_the_tensor(a_mn, b_mn):
    """bf16 operands: the coordinate along the contiguous dimension must be a multiple of 8
    elements. Boxes may hang over the end of the tensor (the fill value is read there), and a
    unit's boxes must fill exactly the bytes its barrier expects."""
    rng = random.Random(2)
    shapes = [(m, n, k) for _, m, n, k in MODEL_SHAPES[:8]] + \
             [(rng.randint(1, 2000), rng.randint(1, 2000), rng.randint(1, 3000)) for _ in range(60)]
    for M, N, K in shapes:
        p = S.plan_gemm(M, N, K)
        for u in list(range(min(p.total_units, 40))) + list(range(max(0, p.total_units - 40), p.total_units)):
            mt, nt, kb, kn, half = S.decode_tile(p, u)
            boxes = S.operand_boxes(p, u, a_mn, b_mn)
            nbytes = {"A": 0, "B": 0}
            for which, x, y, bx, by in boxes:
                assert x % 8 == 0 and x >= 0 and y >= 0
                rows, cols = {"A": (M, K), "B": (N, K)}[which]
                contiguous, other = (rows, cols) if (a_mn if which == "A" else b_mn) else (cols, rows)
                # a load may start past the end of the tensor (the second 128-row box of a tile on
                # the ragged edge does, and so does every box of the second half of such a tile): it
                # reads the fill value and still delivers its bytes. The FIRST box of each operand of
                # a whole tile or a first half starts inside.
                if nbytes[which] == 0 and half <= 0:
                    assert x < contiguous and y < other, (which, x, y, M, N, K)
                nbytes[which] += bx * by * 2
            assert nbytes["A"] == 128 * 64 * 2
            assert nbytes["B"] == (p.bn if half < 0 else p.bn // 2) * 64 * 2
            c0, nc = S.output_columns(p, u)
            assert c0 % 64 == 0 and c0 < -(-N // p.bn) * p.bn


def test_units_of_one_cta_are_strided_by_the_grid_and_balanced():
    for name, M, N, K in MODEL_SHAPES:
        p = S.plan_gemm(M, N, K)
        counts = [len(S.cta_units(p, c)) for c in range(p.grid)]
        assert sum(counts) == p.total_units and max(counts) - min(counts) <= 1
        # in tile-equivalents (a half tile counts 1/2) no CTA carries a whole tile more than another
        load = []
        for c in range(p.grid):
            load.append(sum(1.0 if S.decode_tile(p, u)[4] < 0 else 0.5 for u in S.cta_units(p, c)))
        assert max(load) - min(load) <= 1.0


# ---------------------------------------------------------------------------------------------
# tensor-parallel kernels
# ---------------------------------------------------------------------------------------------
TP_SHAPES = [(4096, 2304), (4096, 4096), (4096, 16384), (8192, 4096), (8192, 1152), (2048, 36728)]


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("mode", [1, 2])
def test_tensor_parallel_units_cover_every_tile_once_on_every_rank(tp, mode):
    for M, N in TP_SHAPES:
        for rank in range(tp):
            p = S.plan_tp(M, N, tp, rank, mode)
            seen = {}
            for u in range(p.total_units):
                mt, nt, half = S.tp_decode_tile(p, u)
                assert 0 <= mt < p.m_tiles and 0 <= nt < p.n_tiles
                for h in ((0, 1) if half < 0 else (half,)):
                    assert (mt, nt, h) not in seen
                    seen[(mt, nt, h)] = u
            assert len(seen) == 2 * p.m_tiles * p.n_tiles


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_a_rank_starts_with_rows_that_need_no_transfer_and_ends_with_its_own_output(tp):
    """All-gather -> GEMM: the first row blocks a rank multiplies are its own slot's, so the tensor
    cores start while the peers' rows are still on their way. GEMM -> reduce-scatter: tiles owned by
    the next rank come first and the rank's own rows last, so what must cross NVLink leaves early."""
    M, N = 8192, 4096
    for rank in range(tp):
        p = S.plan_tp(M, N, tp, rank, 1)
        # (a slot shorter than a group of TP_GROUP_M row blocks shares its group with the next
        # rank's slot: with 8 ranks and 8192 tokens the first wave cannot be all local anyway,
        # 8 x 16 local tiles against 148 CTAs)
        lead = min(p.tiles_per_slot, S.T["TP_GROUP_M"])
        first_rows = {S.tp_decode_tile(p, u)[0] // p.tiles_per_slot for u in range(lead)}
        assert first_rows == {rank}
        q = S.plan_tp(M, N, tp, rank, 2)
        owners = [S.tp_decode_tile(q, u)[0] // q.tiles_per_slot for u in range(q.total_units)]
        assert owners[0] == (rank + 1) % tp
        last_remote = max(i for i, o in enumerate(owners) if o != rank)
        first_own = min(i for i, o in enumerate(owners) if o == rank)
        # groups of TP_GROUP_M row blocks are walked column by column, so own and remote units
        # interleave only inside the one group that holds the slot boundary
        assert last_remote - first_own < S.T["TP_GROUP_M"] * q.n_tiles


def test_a_row_block_never_straddles_two_owners_when_the_host_accepts_the_shape():
    """The fused path is taken only when the token count is a multiple of 128 x tp
    (parallel/fused_tp.py): a 128-row tile then lies inside one rank's slot, which is what lets the
    epilogue of the reduce-scatter kernel pick ONE owner plane per tile."""
    for tp in (2, 4, 8):
        for M in (128 * tp, 4096, 8192, 128 * tp * 7):
            p = S.plan_tp(M, 1024, tp, 0, 2)
            assert (M // tp) % 128 == 0 and p.tiles_per_slot * tp == p.m_tiles
            for mt in range(p.m_tiles):
                lo, hi = mt * 128, mt * 128 + 127
                assert lo // (M // tp) == hi // (M // tp)
