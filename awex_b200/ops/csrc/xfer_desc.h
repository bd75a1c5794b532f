// Descriptor table consumed by the fused transfer kernel.
//
// One descriptor is a 2-D slab: `rows` rows of `row_elems` elements, rows
// `src_stride` / `dst_stride` bytes apart (source rows may instead be gathered
// through a per-row offset table, which is how a quantisation block collects
// rows that a layout permutation scattered), read from this GPU's memory and
// written to `dst`, which is either local or a peer-mapped address of another
// GPU on the same NVLink domain.  The host cuts every slab into tiles of
// `tile_rows` x `tile_cols` elements; tiles of all descriptors are numbered
// consecutively (`tile_begin` is the number of the slab's first tile) and the
// kernel's CTAs split the tile range evenly.
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
constexpr int kLookahead = 4;
constexpr int kThreads = 512;

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
  // optional: descriptor index of the first tile of every chunk of 2^chunk_shift
  // tiles; when given, chunks are dealt round-robin to the CTAs
  const uint32_t* chunk_desc;
  uint32_t chunk_shift;
};

}  // namespace awex
