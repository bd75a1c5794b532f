// Descriptor table consumed by the fused transfer kernel.
//
// One descriptor is a 2-D slab: `rows` rows of `row_elems` elements, rows
// `src_stride` / `dst_stride` bytes apart (source rows may instead be gathered
// through a per-row offset table, which is how a quantisation block collects
// rows that a layout permutation scattered), read from this GPU's memory and
// written to `dst`, which is either local or a peer-mapped address of another
// GPU on the same NVLink domain.  The host cuts every slab into tiles of
// `tile_rows` x `tile_cols` elements; tiles of all descriptors are numbered
// consecutively (`tile_begin` is the number of the slab's first tile).  Which
// tiles a CTA works on is either an even split of the whole range or, when the
// host supplies one, its entry of a per-CTA plan (`CtaPlan`).
//
// The Python encoder (awex_b200/transfer/descriptors.py) mirrors this layout
// with a numpy structured dtype; sizeof is checked at load time.
#pragma once
#include <cstdint>

namespace awex {

enum XferOp : uint32_t {
  OP_COPY = 0,       // raw bytes; row_elems counts bytes
  OP_CAST = 1,       // elementwise dtype conversion
  OP_ADD = 2,        // out = dst_dtype(float(in) + aux_f)
  OP_FP8_BLOCK = 3,  // 128x128 block-scaled e4m3 quantisation, scales to aux_ptr
};

enum XferDtype : uint32_t { DT_BYTES = 0, DT_BF16 = 1, DT_F16 = 2, DT_F32 = 3, DT_FP8_E4M3 = 4 };

enum XferFlags : uint32_t {
  FLAG_BULK = 1u << 0,      // every row chunk is 16-byte aligned and sized on the source side
  FLAG_DST_VEC16 = 1u << 1, // ... and on the destination side
  FLAG_UE8M0 = 1u << 2,     // OP_FP8_BLOCK: round scales up to a power of two
  FLAG_OUT_BULK = 1u << 3,  // OP_FP8_BLOCK, staged, destination rows 16-byte aligned: leave through shared memory and
                            // bulk-async stores (destinations across NVLink, where per-thread stores are limited by
                            // the SM's outstanding writes)
};

struct alignas(16) XferDesc {
  uint64_t src;         //  0
  uint64_t dst;         //  8
  uint64_t rows;        // 16
  uint64_t row_elems;   // 24
  int64_t src_stride;   // 32  bytes
  int64_t dst_stride;   // 40  bytes
  uint64_t tile_begin;  // 48
  uint64_t aux_ptr;     // 56  OP_FP8_BLOCK: address of the scale for block (0,0) of this slab
  int64_t aux_stride;   // 64  OP_FP8_BLOCK: floats between consecutive block rows of scales
  double aux_f;         // 72  OP_ADD: the addend
  uint32_t op;          // 80
  uint32_t flags;       // 84
  uint32_t src_dtype;   // 88
  uint32_t dst_dtype;   // 92
  uint32_t tile_rows;   // 96
  uint32_t tile_cols;   // 100 elements
  uint32_t col_tiles;   // 104 tiles per band of tile_rows rows
  uint32_t reserved;    // 108
  uint64_t row_table;   // 112 optional: address of int64 byte offsets, one per row, replacing row * src_stride
  uint64_t tensor_map;  // 120 optional: address of a 128-byte CUtensorMap over this slab (2-D tiled loads)
};
static_assert(sizeof(XferDesc) == 128, "descriptor layout is shared with the Python encoder");

// Status words written by kernels (int32[4]: code, detail0, detail1, detail2).
enum XferStatus : int32_t {
  ST_OK = 0,
  ST_READY_TIMEOUT = 1,  // a destination never announced that it is ready for this epoch
  ST_LOAD_TIMEOUT = 2,   // a staged load did not complete in time
  ST_FLAG_TIMEOUT = 3,   // a sender's completion flag did not arrive in time
  ST_BAD_DESC = 4,       // a descriptor failed a device-side sanity check
};

constexpr int kStageBytes = 32 * 1024;
constexpr int kStages = 6;
constexpr int kThreads = 512;
constexpr int kFp8Block = 128;  // quantisation block edge

// One CTA's share of the table.  The CTAs of a group (`size` of them, this one
// being number `rank`) own the tile range [tile_begin, tile_end), cut into chunks
// of 2^chunk_shift tiles counted from tile_begin; CTA `rank` takes chunks rank,
// rank + size, rank + 2 size, ...  `chunk_off` is where the group's chunks start
// in XferParams::chunk_desc.  The host makes one group per destination GPU, sized
// in proportion to the destination's bytes, so that every receiver is fed during
// the whole kernel while cheap and expensive tiles are still spread over the
// group's CTAs; one group of all CTAs deals the whole table round-robin, groups
// of one CTA are contiguous ranges.
struct alignas(16) CtaPlan {
  uint64_t tile_begin;
  uint64_t tile_end;
  uint32_t rank;
  uint32_t size;
  uint32_t chunk_off;
  uint32_t reserved;
};
static_assert(sizeof(CtaPlan) == 32, "plan layout is shared with the Python encoder");

struct XferParams {
  const XferDesc* descs;
  uint32_t n_desc;
  uint64_t n_tiles;
  uint64_t epoch;
  // bounded waits
  uint64_t timeout_ns;
  // flags this kernel waits for before it writes: local pad, slots to watch
  const uint64_t* ready_pad;
  const uint32_t* ready_slots;
  uint32_t n_ready;
  // flags this kernel raises when all its writes are done: peer-mapped addresses
  uint64_t* const* done_flags;
  uint32_t n_done;
  // scratch: CTA arrival counter (self-resetting) and status words
  unsigned int* cta_counter;
  int32_t* status;
  // optional: one plan per CTA (gridDim.x entries) and, for every chunk of every
  // group, the index of the descriptor that holds the chunk's first tile.  Without
  // a plan the CTAs split the whole tile range evenly into contiguous ranges.
  const CtaPlan* cta_plan;
  const uint32_t* chunk_desc;
  uint32_t chunk_shift;
};

}  // namespace awex
