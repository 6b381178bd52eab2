"""Host restatement of the GEMM kernels' work decomposition (csrc/gemm_sm100.cu: ``ft_gemm_bf16``
and ``decode_tile``; csrc/gemm_tp_sm100.cu: ``tp_set_tail_split`` and ``tp_decode_tile``): which
work unit covers which output tile, K range and column half, in which order a CTA visits its
units, and which TMA boxes it asks for. Integer arithmetic only, so the index math of every shape
can be checked on the CPU: each output element produced exactly once per K piece, no empty K
piece, box coordinates on 16-byte boundaries and inside what the tensor map describes.

The constants are read from the CUDA sources, so a change there that this model does not follow
fails the tests instead of passing unnoticed."""
from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "forgetrain_b200" / "csrc"


def source_constants(file: str, names: list[str]) -> dict[str, int]:
    text = (CSRC / file).read_text()
    out = {}
    for n in names:
        m = re.search(rf"constexpr int {n} = (\d+);", text)
        assert m, f"{n} not found in {file}"
        out[n] = int(m.group(1))
    return out


G = source_constants("gemm_sm100.cu", ["GEMM_BM", "GEMM_BK", "GEMM_GROUP_M"])
T = source_constants("gemm_tp_sm100.cu", ["TP_BM", "TP_BK", "TP_BN", "TP_GROUP_M", "TP_MAX"])


@dataclass
class Plan:
    M: int
    N: int
    K: int
    bn: int
    splitk: int
    m_tiles: int
    n_tiles: int
    k_iters: int
    split_from: int
    total_units: int
    grid: int
    out_mode: str        # "bf16" | "f32" | "f32_add"


def plan_gemm(M: int, N: int, K: int, out_f32: bool = False, accumulate: bool = False,
              splitk: int = 0, bn: int = 0, max_ctas: int = 148, sms: int = 148) -> Plan:
    """``ft_gemm_bf16`` up to the launch."""
    assert M > 0 and N > 0 and K > 0 and not (accumulate and not out_f32)
    if max_ctas <= 0 or max_ctas > sms:
        max_ctas = sms
    k_iters = -(-K // G["GEMM_BK"])
    if bn not in (128, 256):
        bn = 128 if N <= 128 else 256
    m_tiles, n_tiles = -(-M // G["GEMM_BM"]), -(-N // bn)
    if not out_f32:
        splitk = 1
    if splitk <= 0:
        tiles = m_tiles * n_tiles
        splitk = 1
        if tiles < max_ctas:
            splitk = max_ctas // tiles
            splitk = min(splitk, max(k_iters // 8, 1), 16)
    splitk = max(1, min(splitk, k_iters))
    total = m_tiles * n_tiles * splitk
    split_from, total_units = total, total
    if bn == 256 and splitk == 1 and max_ctas >= 2:
        rem = total % max_ctas
        if rem > 0 and 2 * rem <= max_ctas:
            split_from, total_units = total - rem, total + rem
    mode = "bf16" if not out_f32 else ("f32_add" if (accumulate or splitk > 1) else "f32")
    return Plan(M, N, K, bn, splitk, m_tiles, n_tiles, k_iters, split_from, total_units,
                max(1, min(total_units, max_ctas)), mode)


def decode_tile(p: Plan, tile: int) -> tuple[int, int, int, int, int]:
    """``(mt, nt, kb, kn, half)`` of work unit ``tile``; ``half`` is -1 for a whole tile."""
    half = -1
    if tile >= p.split_from:
        t = tile - p.split_from
        half = t & 1
        tile = p.split_from + (t >> 1)
    per_split = p.m_tiles * p.n_tiles
    ks, r = divmod(tile, per_split)
    group_sz = G["GEMM_GROUP_M"] * p.n_tiles
    g = r // group_sz
    first_m = g * G["GEMM_GROUP_M"]
    gm = min(p.m_tiles - first_m, G["GEMM_GROUP_M"])
    inn = r - g * group_sz
    mt, nt = first_m + inn % gm, inn // gm
    base, rem = divmod(p.k_iters, p.splitk)
    kb = ks * base + min(ks, rem)
    kn = base + (1 if ks < rem else 0)
    return mt, nt, kb, kn, half


def cta_units(p: Plan, cta: int) -> list[int]:
    return list(range(cta, p.total_units, p.grid))


def operand_boxes(p: Plan, tile: int, a_mn: bool, b_mn: bool) -> list[tuple[str, int, int, int, int]]:
    """``(map, x, y, box_x, box_y)`` in elements for every TMA load of one K step (ki = kb) of a unit:
    x is the coordinate along the contiguous dimension of the tensor in memory."""
    mt, nt, kb, kn, half = decode_tile(p, tile)
    BM, BK, bn = G["GEMM_BM"], G["GEMM_BK"], p.bn
    out = []
    if not a_mn:
        out.append(("A", kb * BK, mt * BM, BK, BM))
    else:
        for lane in range(BM // 64):
            out.append(("A", mt * BM + lane * 64, kb * BK, 64, BK))
    nB = bn // 64 if b_mn else bn // 128
    nBt = nB if half < 0 else nB // 2
    jb0 = 0 if half <= 0 else nB // 2
    for j in range(nBt):
        if not b_mn:
            out.append(("B", kb * BK, nt * bn + (jb0 + j) * 128, BK, 128))
        else:
            out.append(("B", nt * bn + (jb0 + j) * 64, kb * BK, 64, BK))
    return out


def output_columns(p: Plan, tile: int) -> tuple[int, int]:
    """First column and number of columns of the accumulator a unit drains."""
    _, nt, _, _, half = decode_tile(p, tile)
    ncols = p.bn if half < 0 else p.bn // 2
    return nt * p.bn + (p.bn // 2 if half > 0 else 0), ncols


# ---------------------------------------------------------------------------------------------
# tensor-parallel kernels
# ---------------------------------------------------------------------------------------------
@dataclass
class TpPlan:
    M: int
    N: int
    tp: int
    rank: int
    mode: int            # 1: all-gather -> GEMM, 2: GEMM -> reduce-scatter
    m_tiles: int
    n_tiles: int
    tiles_per_slot: int
    split_from: int
    total_units: int
    grid: int

    @property
    def rot(self) -> int:
        first = self.rank if self.mode == 1 else (self.rank + 1) % self.tp
        return first * self.tiles_per_slot


def plan_tp(M: int, N: int, tp: int, rank: int, mode: int, grid: int = 148) -> TpPlan:
    assert 2 <= tp <= T["TP_MAX"] and M % tp == 0
    slot_rows = M // tp
    m_tiles, n_tiles = -(-M // T["TP_BM"]), -(-N // T["TP_BN"])
    total = m_tiles * n_tiles
    split_from = total_units = total
    rem = total % grid
    if grid >= 2 and rem > 0 and 2 * rem <= grid:
        split_from, total_units = total - rem, total + rem
    return TpPlan(M, N, tp, rank, mode, m_tiles, n_tiles, -(-slot_rows // T["TP_BM"]), split_from,
                  total_units, grid)


def tp_decode_tile(p: TpPlan, tile: int) -> tuple[int, int, int]:
    half = -1
    if tile >= p.split_from:
        t = tile - p.split_from
        half = t & 1
        tile = p.split_from + (t >> 1)
    group_sz = T["TP_GROUP_M"] * p.n_tiles
    g = tile // group_sz
    first_m = g * T["TP_GROUP_M"]
    gm = min(p.m_tiles - first_m, T["TP_GROUP_M"])
    inn = tile - g * group_sz
    ml, nt = first_m + inn % gm, inn // gm
    return (ml + p.rot) % p.m_tiles, nt, half
