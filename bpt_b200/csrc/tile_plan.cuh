// Record layout of the tensor-core path's tile plan, shared by the host planner and the kernel.
#pragma once

#include "common.cuh"

namespace bpt {

constexpr int kTileRows = 16;    // destination rows per tile (one mma M block)
constexpr int kTileChunk = 64;   // source columns processed per inner step; column counts are padded to it
constexpr int kTileInts = 40;    // int32 words per tile record
constexpr int kTileRowOff = 0;   // [0,16): destination row ids, -1 = unused
constexpr int kTileSlotOff = 16; // [16,32): partial-result slot per row, -1 = the tile holds the whole row
constexpr int kTileNcolsPad = 32;
constexpr int kTileColOff = 33;  // offset of the tile's column list in `cols`
constexpr int kTileEtOff = 34;   // offset of the tile's [16][ncols_pad] edge-type matrix in `et`
constexpr int kTileTq = 35;      // edge types [0, tq) occur in the tile (multiple of 8)
constexpr int kTileNcols = 36;   // columns before padding
constexpr uint16_t kNoEdge = 0xFFFF;

}  // namespace bpt
