"""CPU: the index arithmetic of two device-side schemes, restated in Python and checked exhaustively on small cases
(the kernels themselves are checked bit for bit on the GPU in tests/test_gpu_gemm.py).

1. The symmetric tile enumeration of the grouped GEMM (csrc/gemm_common.cuh, get_tile with sym_rows > 0) together
   with the rule of the epilogue that stores a chunk a second time, transposed (csrc/gemm.cu): every element of
   every group must be written exactly once.
2. The swizzled 64 x 64 transposing tile of csrc/muon.cu (TransposeTile)."""
import numpy as np
import pytest

TILE = 256     # B200MOE_TILE_M: granularity of the transposed-store rule


def _sym_tiles(R, TM, TN):
    """(m0, n0) of the tiles one group of R rows x R columns runs, in the kernel's order."""
    nt = (R + TN - 1) // TN
    per = sum(nt - (mi * TM) // TN for mi in range((R + TM - 1) // TM))
    out = []
    for tile in range(per):
        r, mi = tile, 0
        while True:
            ln = nt - (mi * TM) // TN
            if r < ln:
                break
            r -= ln
            mi += 1
        out.append((mi * TM, ((mi * TM) // TN + r) * TN))
    return out


@pytest.mark.parametrize("R,TM,TN", [(256, 256, 256), (1536, 256, 256), (2048, 256, 256), (1024, 128, 256)])
def test_symmetric_enumeration_and_transposed_chunks_cover_every_element_once(R, TM, TN):
    written = np.zeros((R, R), dtype=np.int32)
    for m0, n0 in _sym_tiles(R, TM, TN):
        for row0 in range(m0, min(m0 + TM, R), 32):            # one epilogue warp: 32 rows
            for c in range(n0, min(n0 + TN, R), 64):            # one chunk: 64 columns
                written[row0:row0 + 32, c:c + 64] += 1
                if c // TILE > row0 // TILE:                    # right of the diagonal tile: store the transpose too
                    written[c:c + 64, row0:row0 + 32] += 1
    assert (written == 1).all()


def test_swizzled_transpose_tile():
    src = np.arange(64 * 64).reshape(64, 64)
    words = np.zeros(64 * 32 * 2, dtype=np.int64)               # 64 rows of 32 words, two values per word
    for v in range(512):                                        # put(): vector of row v >> 3 at column 8 * (v & 7)
        r, c8 = v >> 3, (v & 7) * 8
        base = r * 32 + ((c8 >> 1) ^ ((r >> 3) << 2))
        assert base % 4 == 0                                    # 16-byte vectors stay whole and aligned
        words[2 * base:2 * base + 8] = src[r, c8:c8 + 8]
    dst = np.zeros((64, 64), dtype=np.int64)
    for v in range(512):                                        # get_transposed()
        r, c8 = v >> 3, (v & 7) * 8
        banks = set()
        for j in range(8):
            sr = c8 + j
            w = sr * 32 + ((r >> 1) ^ ((sr >> 3) << 2))
            dst[r, c8 + j] = words[2 * w + (r & 1)]
            banks.add(w % 32)
        assert len(banks) == 1                                  # one lane walks one bank ...
    assert (dst == src.T).all()
    # ... and the 8 lanes that share a destination row chunk pattern (same r, different c8) hit 8 different banks
    for r in range(64):
        for j in range(8):
            assert len({((c8 + j) * 32 + ((r >> 1) ^ (((c8 + j) >> 3) << 2))) % 32 for c8 in range(0, 64, 8)}) == 8


def test_slots_without_a_row_are_skipped_by_the_combine_model():
    """An expert index outside [0, E) leaves its slot without a row: the rank pass writes -1 into slot_row /
    slot_pos and every consumer skips such entries (csrc/permute.cu, csrc/combine.cu, csrc/ep.cu).  The CPU model
    of the combine follows the same rule."""
    import torch
    from tests.cpu_kernels import CpuKernels
    rows = torch.arange(12, dtype=torch.float32).view(6, 2)
    table = torch.tensor([0, -1, 5, 2], dtype=torch.int32)          # T = 2, k = 2; token 0's second slot has no row
    w = torch.tensor([[0.5, 100.0], [1.0, 2.0]])
    out = CpuKernels.combine_raw(rows, w, table, 2, 2)
    assert torch.equal(out[0], 0.5 * rows[0])
    assert torch.equal(out[1], rows[5] + 2.0 * rows[2])
    assert torch.equal(CpuKernels.combine_raw(rows, None, table, 2, 2)[0], rows[0])


def test_expert_parallel_plan_blocks_tile_every_segment_and_overflow_is_decided_alike():
    """The plan of the expert-parallel exchange (model of csrc/ep.cu ep_plan_kernel): the blocks of the W sources
    tile each expert's live rows without gap or overlap, the home rank's idea of where its rows go (dest_base) is the
    owner's idea of where that source's block starts (src_base), and a count matrix that does not fit a fixed
    capacity is refused by every rank together."""
    import torch
    from tests.cpu_kernels import CpuKernels
    g = torch.Generator().manual_seed(0)
    W, E = 4, 16
    El = E // W
    counts = torch.randint(0, 700, (W, E), generator=g)
    counts[:, 5] = 0                                              # an expert nobody routes to
    plans = [CpuKernels.ep_plan(counts, W, r, E) for r in range(W)]
    for owner in range(W):
        p = plans[owner]
        for j in range(El):
            e = owner * El + j
            lo = int(p["poffs_l"][j])
            assert lo % 256 == 0 and int(p["poffs_l"][j + 1]) - lo == (int(p["counts_l"][j]) + 255) // 256 * 256
            at = lo
            for s in range(W):
                assert int(p["src_base"][s * El + j]) == at == int(plans[s]["dest_base"][e])
                at += int(counts[s, e])
            assert at == lo + int(p["counts_l"][j])
    rows = [int(p["poffs_l"][El]) for p in plans]
    cap = max(rows) - 256                                         # one owner does not fit
    refused = [CpuKernels.ep_plan(counts, W, r, E, rows_cap=cap) for r in range(W)]
    assert all(p["overflow"] for p in refused)
    assert all(int(p["poffs_l"].sum()) == 0 and int(p["counts_l"].sum()) == 0 and (p["src_base"] < 0).all() for p in refused)
    assert not any(CpuKernels.ep_plan(counts, W, r, E, rows_cap=max(rows))["overflow"] for r in range(W))

