// Record layout of the tensor-core path's tile plan, shared by the planners (host and device) and the kernels.
//
// A *group* is a sorted list of source columns (padded to a multiple of 64) plus up to
// kMaxMBlocks *m-blocks*; an m-block is <=16 destination rows with a dense matrix of edge
// types over the group's columns (kNoEdge = no edge in that cell).  One thread block stages
// the group's K/V rows once per head and every m-block (one warp each) attends over them.
#pragma once

#include "common.cuh"

namespace bpt {

constexpr int kTileRows = 16;     // destination rows per m-block (one mma M block)
constexpr int kTileChunk = 64;    // source columns per pipeline step; column counts are padded to it
constexpr int kMaxMBlocks = 8;    // m-blocks (warps) per group at most
constexpr int kMaskCols = 32;     // an m-block's activity mask has one bit per 32 columns
constexpr int kMaxMaskBits = 32;  // so a group holds at most 1024 columns

// group record: kGroupInts int32 words
constexpr int kGroupInts = 8;
constexpr int kGroupColOff = 0;    // offset of the column list in `cols`
constexpr int kGroupNcolsPad = 1;  // padded column count (multiple of kTileChunk, may be 0)
constexpr int kGroupMbFirst = 2;   // first m-block record
constexpr int kGroupMbCount = 3;
constexpr int kGroupNcols = 4;     // columns before padding

// m-block record: kMbInts int32 words
constexpr int kMbInts = 56;
constexpr int kMbRowOff = 0;       // [0,16): destination row ids, -1 = unused
constexpr int kMbSlotOff = 16;     // [16,32): partial-result slot per row, -1 = this m-block holds the whole row
constexpr int kMbRowEtOff = 32;    // [32,48): the row's single edge type when kMbQrSlot < 0
constexpr int kMbEtOff = 48;       // offset (in cells) of the [chunks][16][64] edge-type matrix in `et`
constexpr int kMbChunkMask = 49;   // bit s set = some row has an edge in columns [32 s, 32 s + 32)
constexpr int kMbTq = 50;          // edge types [0, tq) occur (multiple of 8)
constexpr int kMbFineMask = 52;    // bit s set = some row has an edge in columns [16 s, 16 s + 16); meaningful for groups of
                                   // at most 512 columns (the tcgen05 kernels' plans), 0 beyond
constexpr int kMbQrSlot = 51;      // >= 0: needs the per-row relative-position table, in this shared-memory
                                   // slot; -1: every row's edges share one type, so the term is a per-row
                                   // constant that cancels in the softmax and only shifts lse
// Exported cell payloads (edge positions) are stored per 64-column chunk in the order the mma
// lanes consume them rather than row by row: cell (r, c) of a chunk sits at
//   (((c / 32) * 4 + (c % 32) / 8) * 32 + lane) * 4 + (r / 8) * 2 + (c & 1),   lane = (r % 8) * 4 + (c % 8) / 2,
// so lane (g, t) finds {(g, c), (g, c+1), (g+8, c), (g+8, c+1)} for c = 32 half + 8 nt + 2t in one
// 16-byte piece, and the 32 lanes' pieces of one (half, nt) are contiguous.
__host__ __device__ constexpr int cell_pos_index(int r, int c) {
    return (((c / 32) * 4 + (c % 32) / 8) * 32 + (r % 8) * 4 + (c % 8) / 2) * 4 + (r / 8) * 2 + (c & 1);
}
// Row stride (in 16-bit entries) of the per-warp score tables of the tile kernels: t_max types and the -inf
// entry, padded.  t_max + 10 is an odd number of 32-bit words, which spreads a table's 16 rows over the
// shared-memory banks (worth ~15 % of the forward on narrow tiles); t_max + 8 saves 512 bytes per block and
// is taken when exactly those bytes would stop a second block per SM (plans whose widest tile has 192
// columns).  other_bytes = the block's shared memory without the tables; n_tables = warps per block.
inline int table_stride(size_t other_bytes, int t_max, int n_tables) {
    constexpr size_t kTwoBlocksPerSm = (228 * 1024 - 2 * 1024) / 2;  // per block, with the 1 KB the system reserves
    const size_t wide = other_bytes + static_cast<size_t>(n_tables) * kTileRows * (t_max + 10) * 2;
    const size_t narrow = other_bytes + static_cast<size_t>(n_tables) * kTileRows * (t_max + 8) * 2;
    return wide > kTwoBlocksPerSm && narrow <= kTwoBlocksPerSm ? t_max + 8 : t_max + 10;
}
constexpr uint16_t kNoEdge = 0xFFFF;
constexpr uint8_t kNoEdge8 = 0xFF;

}  // namespace bpt
