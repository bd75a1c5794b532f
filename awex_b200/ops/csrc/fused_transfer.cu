// Fused resharding transfer for sm_100a.
//
// One persistent launch per (update, source GPU) walks a descriptor table
// (xfer_desc.h).  Which tiles a CTA works on comes from its entry of a per-CTA
// plan the host builds (one group of CTAs per destination GPU, round-robin
// chunks of tiles inside a group), or, without a plan, from an even split of
// the tile range.  A tile is staged from this GPU's HBM into shared memory with
// bulk-async copies (cp.async.bulk global->shared, or one tiled
// cp.async.bulk.tensor load where the slab has a tensor map; completion on an
// mbarrier) through a ring of 32 KiB stages, then leaves either
//   * unchanged, by bulk-async copies shared->global whose destination may be a
//     peer GPU's memory mapped over NVLink (pure layout moves: slices, row
//     permutations, column slabs), or
//   * transformed in registers (dtype cast, constant add, 128x128 block-scaled
//     fp8 e4m3 quantisation) and stored with 16-byte vector stores.
// All loads read local memory; remote memory is only ever written.
// When every CTA has drained its stores, the last one raises a per-destination
// flag (release, system scope) carrying the update's epoch; receivers wait on
// those flags with a bounded spin (wait_flags_kernel).  Every wait in this file
// has a deadline after which the kernel records a status and returns.
//
// The reference does the same work with one ATen copy/cast kernel per slab,
// an all-gather per fused QKV, and one NCCL send/recv pair per slab
// (awex/transfer/nccl_comm.py:378-624, awex/converter/mcore_converter.py:1040-1052).

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "fp8_math.cuh"
#include "xfer_desc.h"

namespace awex {

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// global -> shared, completion counted in bytes on an mbarrier of this CTA
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
// shared -> global (local or peer-mapped), tracked by the thread's bulk group
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---------------------------------------------------------------- element helpers
__device__ __forceinline__ uint32_t dtype_size(uint32_t dt) {
  return dt == DT_F32 ? 4u : (dt == DT_BF16 || dt == DT_F16) ? 2u : 1u;
}
__device__ __forceinline__ float load_as_float(const unsigned char* p, uint32_t dt) {
  switch (dt) {
    case DT_BF16: return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
    case DT_F16: return __half2float(*reinterpret_cast<const __half*>(p));
    case DT_F32: return *reinterpret_cast<const float*>(p);
    case DT_FP8_E4M3: {
      __half_raw h = __nv_cvt_fp8_to_halfraw(*p, __NV_E4M3);
      return __half2float(*reinterpret_cast<__half*>(&h));
    }
    default: return static_cast<float>(*p);
  }
}
__device__ __forceinline__ void store_from_float(unsigned char* p, uint32_t dt, float v) {
  switch (dt) {
    case DT_BF16: *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(v); break;
    case DT_F16: *reinterpret_cast<__half*>(p) = __float2half_rn(v); break;
    case DT_F32: *reinterpret_cast<float*>(p) = v; break;
    case DT_FP8_E4M3: *p = static_cast<unsigned char>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3)); break;
    default: *p = static_cast<unsigned char>(v); break;
  }
}

// Position of a tile inside its slab.
struct Tile {
  uint64_t row0;
  uint32_t rows;
  uint64_t col0;  // elements
  uint32_t cols;  // elements
  uint32_t band, ct;
};
__device__ __forceinline__ Tile tile_of(const XferDesc& d, uint64_t k) {
  Tile t;
  if (k <= 0xFFFFFFFFull) {  // the common case: a 32-bit division
    const uint32_t k32 = static_cast<uint32_t>(k);
    t.band = k32 / d.col_tiles;
    t.ct = k32 - t.band * d.col_tiles;
  } else {
    t.band = static_cast<uint32_t>(k / d.col_tiles);
    t.ct = static_cast<uint32_t>(k % d.col_tiles);
  }
  t.row0 = static_cast<uint64_t>(t.band) * d.tile_rows;
  t.col0 = static_cast<uint64_t>(t.ct) * d.tile_cols;
  uint64_t r = d.rows - t.row0;
  uint64_t c = d.row_elems - t.col0;
  t.rows = r < d.tile_rows ? static_cast<uint32_t>(r) : d.tile_rows;
  t.cols = c < d.tile_cols ? static_cast<uint32_t>(c) : d.tile_cols;
  return t;
}
__device__ __forceinline__ uint32_t stage_pitch(const XferDesc& d) {
  return (d.tile_cols * dtype_size(d.src_dtype) + 15u) & ~15u;
}

// Byte offset of source row `row` of a slab from its `src` address.
__device__ __forceinline__ int64_t src_row_offset(const XferDesc& d, uint64_t row) {
  if (d.row_table) return reinterpret_cast<const int64_t*>(d.row_table)[row];
  return static_cast<int64_t>(row) * d.src_stride;
}

// Descriptor cursor: tile number -> (descriptor, tile inside it), advanced monotonically.
struct Cursor {
  uint32_t di;
  uint64_t begin, end;  // tile range of descs[di]
};
__device__ __forceinline__ void cursor_seek(Cursor& c, const XferParams& p, uint64_t tile) {
  uint32_t lo = 0, hi = p.n_desc - 1;
  while (lo < hi) {  // last descriptor whose tile_begin <= tile
    uint32_t mid = (lo + hi + 1) >> 1;
    if (p.descs[mid].tile_begin <= tile) lo = mid; else hi = mid - 1;
  }
  c.di = lo;
  c.begin = p.descs[lo].tile_begin;
  c.end = (lo + 1 < p.n_desc) ? p.descs[lo + 1].tile_begin : p.n_tiles;
}
// Jump to the descriptor that holds the first tile of a chunk (host-built index).
__device__ __forceinline__ void cursor_jump(Cursor& c, const XferParams& p, uint64_t chunk) {
  c.di = p.chunk_desc[chunk];
  c.begin = p.descs[c.di].tile_begin;
  c.end = (c.di + 1 < p.n_desc) ? p.descs[c.di + 1].tile_begin : p.n_tiles;
}
__device__ __forceinline__ void cursor_advance_to(Cursor& c, const XferParams& p, uint64_t tile) {
  while (tile >= c.end) {
    ++c.di;
    c.begin = c.end;
    c.end = (c.di + 1 < p.n_desc) ? p.descs[c.di + 1].tile_begin : p.n_tiles;
  }
}

// ---------------------------------------------------------------- tile bodies
// Every body that all warps take part in contains exactly one CTA-wide barrier,
// placed after the thread's last read of the staged tile.  The barrier also
// carries the abort vote (`__syncthreads_or`): a thread whose bounded wait ran
// out votes to stop, and every thread leaves the tile loop at the same point.

// Elementwise path straight from global memory (unaligned slabs, rare dtypes).
__device__ bool tile_elementwise_global(const XferDesc& d, const Tile& t, uint32_t my_abort) {
  const uint32_t ses = dtype_size(d.src_dtype), des = dtype_size(d.dst_dtype);
  const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src);
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst);
  const uint64_t n = static_cast<uint64_t>(t.rows) * t.cols;
  const float addend = d.op == OP_ADD ? static_cast<float>(d.aux_f) : 0.f;
  for (uint64_t e = threadIdx.x; e < n; e += blockDim.x) {
    uint32_t r = static_cast<uint32_t>(e / t.cols), c = static_cast<uint32_t>(e % t.cols);
    const unsigned char* s = src + src_row_offset(d, t.row0 + r) + (t.col0 + c) * ses;
    unsigned char* o = dst + (t.row0 + r) * d.dst_stride + (t.col0 + c) * des;
    if (d.op == OP_COPY) *o = *s;
    else store_from_float(o, d.dst_dtype, load_as_float(s, d.src_dtype) + addend);
  }
  return __syncthreads_or(static_cast<int>(my_abort)) != 0;
}

// 16 staged bytes -> floats.  kSrc is an XferDtype with 2- or 4-byte elements.
template <uint32_t kSrc>
__device__ __forceinline__ void chunk_to_floats(const uint4& raw, float* v) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if constexpr (kSrc == DT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(w[i]);
  } else if constexpr (kSrc == DT_BF16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}

// kN floats -> destination elements at `o` (aligned to kN * element size, at most 32 bytes).
template <uint32_t kDst, int kN>
__device__ __forceinline__ void floats_to_dst(const float* v, unsigned char* o) {
  if constexpr (kDst == DT_F32) {
#pragma unroll
    for (int i = 0; i < kN; i += 4) *reinterpret_cast<float4*>(o + 4 * i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
    uint32_t packed[kN / 2];
#pragma unroll
    for (int i = 0; i < kN / 2; ++i) {
      if constexpr (kDst == DT_BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        packed[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    if constexpr (kN == 8) *reinterpret_cast<uint4*>(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    else *reinterpret_cast<uint2*>(o) = make_uint2(packed[0], packed[1]);
  }
}

// Cast / add of a staged tile, one 16-byte chunk of the source per thread and
// step: vector load from shared memory, packed converts, 16-byte stores.  Rows
// and chunks advance incrementally; nothing is divided per element.
template <uint32_t kSrc, uint32_t kDst>
__device__ __forceinline__ void cast_chunks(const XferDesc& d, const Tile& t, const unsigned char* stage, float addend) {
  constexpr uint32_t kSes = kSrc == DT_F32 ? 4u : 2u, kDes = kDst == DT_F32 ? 4u : 2u;
  constexpr int kN = 16 / kSes;                    // elements per chunk
  const uint32_t pitch = stage_pitch(d);
  const uint32_t cpr = (t.cols * kSes) >> 4;       // chunks per row (the bulk path keeps rows a multiple of 16 bytes)
  const uint32_t total = t.rows * cpr;
  const uint32_t step_rows = blockDim.x / cpr, step_chunks = blockDim.x % cpr;
  uint32_t row = threadIdx.x / cpr, chunk = threadIdx.x % cpr;
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst) + t.row0 * d.dst_stride + t.col0 * kDes;
  for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + row * pitch + chunk * 16u);
    float v[kN];
    chunk_to_floats<kSrc>(raw, v);
#pragma unroll
    for (int i = 0; i < kN; ++i) v[i] += addend;
    floats_to_dst<kDst, kN>(v, dst + static_cast<int64_t>(row) * d.dst_stride + chunk * (kN * kDes));
    row += step_rows;
    chunk += step_chunks;
    if (chunk >= cpr) {
      chunk -= cpr;
      ++row;
    }
  }
}

template <uint32_t kSrc>
__device__ __forceinline__ bool cast_chunks_from(const XferDesc& d, const Tile& t, const unsigned char* stage, float addend) {
  switch (d.dst_dtype) {
    case DT_F32: cast_chunks<kSrc, DT_F32>(d, t, stage, addend); return true;
    case DT_BF16: cast_chunks<kSrc, DT_BF16>(d, t, stage, addend); return true;
    case DT_F16: cast_chunks<kSrc, DT_F16>(d, t, stage, addend); return true;
    default: return false;
  }
}

// Elementwise path from a staged tile.  Returns the CTA's abort vote.
__device__ bool tile_elementwise_staged(const XferDesc& d, const Tile& t, const unsigned char* stage, uint32_t my_abort) {
  if (!my_abort) {
    const float addend = d.op == OP_ADD ? static_cast<float>(d.aux_f) : 0.f;
    bool done = false;
    if (d.flags & FLAG_DST_VEC16) {
      if (d.src_dtype == DT_BF16) done = cast_chunks_from<DT_BF16>(d, t, stage, addend);
      else if (d.src_dtype == DT_F16) done = cast_chunks_from<DT_F16>(d, t, stage, addend);
      else if (d.src_dtype == DT_F32) done = cast_chunks_from<DT_F32>(d, t, stage, addend);
    }
    if (!done) {  // one-byte types or a destination that is not 16-byte aligned: element by element
      const uint32_t ses = dtype_size(d.src_dtype), des = dtype_size(d.dst_dtype);
      const uint32_t pitch = stage_pitch(d);
      unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst);
      const uint32_t n = t.rows * t.cols;
      for (uint32_t e = threadIdx.x; e < n; e += blockDim.x) {
        uint32_t r = e / t.cols, c = e % t.cols;
        float v = load_as_float(stage + r * pitch + c * ses, d.src_dtype) + addend;
        store_from_float(dst + (t.row0 + r) * d.dst_stride + (t.col0 + c) * des, d.dst_dtype, v);
      }
    }
  }
  return __syncthreads_or(static_cast<int>(my_abort)) != 0;
}

// ---- block fp8 tiles -------------------------------------------------------------------------
// A tile is one 128x128 (or smaller edge) block.

__device__ __forceinline__ void store_scale(const XferDesc& d, const Tile& t, float scale) {
  if (threadIdx.x == 0) reinterpret_cast<float*>(d.aux_ptr)[static_cast<int64_t>(t.band) * d.aux_stride + t.ct] = scale;
}

// Does a quantised tile leave through shared memory and bulk-async stores?
__device__ __forceinline__ bool fp8_leaves_through_stage(const XferDesc& d, const Tile& t) {
  return (d.flags & FLAG_OUT_BULK) != 0 && (d.flags & FLAG_BULK) != 0 && (t.cols & 15u) == 0;
}

// Fast form: 2-byte source staged in shared memory with a 256-byte pitch
// (tile_cols == 128), destination rows 8-byte aligned.  One pass over the stage:
// a thread keeps its 16-byte chunks in registers from the maximum search, the
// CTA agrees on the block maximum with one barrier (`red` is double-buffered by
// the caller, so no second barrier protects it), and the values are quantised
// from the registers.  After the barrier nobody reads the stage any more.
template <int kT, bool kBf16>
__device__ __forceinline__ bool tile_fp8_staged(const XferDesc& d, const Tile& t, const unsigned char* stage, uint32_t* red,
                                                uint32_t my_abort) {
  constexpr int kPasses = (kFp8Block * kFp8Block * 2 / 16) / kT;  // chunks per thread: 8 (256 threads) or 4 (512)
  constexpr uint32_t kRowStep = kT / 16;
  const uint32_t chunk = threadIdx.x & 15u, row0 = threadIdx.x >> 4;
  const bool col_ok = chunk < (t.cols >> 3) && !my_abort;  // the bulk path guarantees cols % 8 == 0
  uint4 raw[kPasses];
  uint32_t m = 0;
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const uint32_t row = row0 + p * kRowStep;
    raw[p] = (col_ok && row < t.rows) ? *reinterpret_cast<const uint4*>(stage + row * 256u + chunk * 16u) : make_uint4(0, 0, 0, 0);
    m = amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(m, raw[p].x), raw[p].y), raw[p].z), raw[p].w);
  }
  m = __reduce_max_sync(0xffffffffu, max(m & 0xFFFFu, m >> 16));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  if (__syncthreads_or(static_cast<int>(my_abort))) return true;
  uint32_t all = red[0];
#pragma unroll
  for (int w = 1; w < kT / 32; ++w) all = max(all, red[w]);
  const float amax = kBf16 ? __uint_as_float(all << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(all)));
  const QuantScale q = make_quant_scale(amax, (d.flags & FLAG_UE8M0) != 0);
  store_scale(d, t, q.s);
  if (fp8_leaves_through_stage(d, t)) {
    // Every thread holds its part of the tile in registers (the barrier above), so the stage can take the
    // result: 128 bytes per row, which warp 0 then sends with one bulk-async store per row.
    unsigned char* out_stage = const_cast<unsigned char*>(stage) + chunk * 8u;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const uint32_t row = row0 + p * kRowStep;
      if (!col_ok || row >= t.rows) continue;
      *reinterpret_cast<uint2*>(out_stage + row * kFp8Block) = quant_chunk16<kBf16>(raw[p], q);
    }
    fence_proxy_async();  // these generic-proxy writes before the bulk stores' async-proxy reads
    __syncthreads();
    return false;
  }
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst) + t.row0 * d.dst_stride + t.col0 + chunk * 8u;
  const bool vec = (d.flags & FLAG_DST_VEC16) != 0;
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const uint32_t row = row0 + p * kRowStep;
    if (!col_ok || row >= t.rows) continue;
    const uint2 out = quant_chunk16<kBf16>(raw[p], q);
    unsigned char* o = dst + static_cast<int64_t>(row) * d.dst_stride;
    if (vec) {
      *reinterpret_cast<uint2*>(o) = out;
    } else {
      const unsigned char* b = reinterpret_cast<const unsigned char*>(&out);
      for (int j = 0; j < 8; ++j) o[j] = b[j];
    }
  }
  return false;
}

// General form: any source dtype and alignment, rows read from global memory
// (directly or through the row table), columns masked at the edge.  Two passes
// over global memory (the second one mostly hits L2).
__device__ bool tile_fp8_generic(const XferDesc& d, const Tile& t, uint32_t* red, uint32_t my_abort) {
  const uint32_t ses = dtype_size(d.src_dtype);
  const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src) + t.col0 * ses;
  const uint32_t chunks = (t.cols + 7u) >> 3;
  const uint32_t items = t.rows * chunks;
  uint32_t m = 0;
  for (uint32_t it = threadIdx.x; it < items; it += blockDim.x) {
    const uint32_t row = it / chunks, c0 = (it % chunks) * 8u;
    const unsigned char* s = src + src_row_offset(d, t.row0 + row) + c0 * ses;
    for (uint32_t j = 0; j < 8u && c0 + j < t.cols; ++j) m = amax_bits_f32(m, load_as_float(s + j * ses, d.src_dtype));
  }
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  if (__syncthreads_or(static_cast<int>(my_abort))) return true;
  uint32_t all = 0;
  for (uint32_t w = 0; w < (blockDim.x >> 5); ++w) all = max(all, red[w]);
  const QuantScale q = make_quant_scale(__uint_as_float(all), (d.flags & FLAG_UE8M0) != 0);
  store_scale(d, t, q.s);
  unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst) + t.row0 * d.dst_stride + t.col0;
  for (uint32_t it = threadIdx.x; it < items; it += blockDim.x) {
    const uint32_t row = it / chunks, c0 = (it % chunks) * 8u;
    const unsigned char* s = src + src_row_offset(d, t.row0 + row) + c0 * ses;
    unsigned char* o = dst + static_cast<int64_t>(row) * d.dst_stride + c0;
    for (uint32_t j = 0; j < 8u && c0 + j < t.cols; j += 2) {
      const float a = load_as_float(s + j * ses, d.src_dtype);
      const bool pair = c0 + j + 1 < t.cols;
      const float b = pair ? load_as_float(s + (j + 1) * ses, d.src_dtype) : 0.f;
      const uint32_t out = quant_pair(a, b, q);
      o[j] = static_cast<unsigned char>(out & 0xFFu);
      if (pair) o[j + 1] = static_cast<unsigned char>(out >> 8);
    }
  }
  return false;
}

// ---------------------------------------------------------------- the kernel
__device__ __forceinline__ bool wants_stage(const XferDesc& d) { return (d.flags & FLAG_BULK) != 0; }

// Bounded wait for a phase of an mbarrier; false when the deadline passed.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint64_t timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity))
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  return true;
}

// Ring of kS stages.  Warp 0 is the copy engine's driver: it issues every load
// and, for pure copies, the stores; all warps work on computed tiles.  Only warp
// 0 watches the stages' mbarriers (the other warps skip copied tiles and may be
// many tiles ahead of the loads, where a stage's phase parity means nothing).
// For a computed tile it then arrives on `ready_bar`, whose phases count staged
// computed tiles only and which the other warps wait on (suspended by the
// hardware, not polling) before they read the stage: between two of its phases
// lies the tile's CTA-wide barrier, so no warp is ever more than one phase away.
// A warp that has passed the barrier of a computed tile less than one ring
// round ago knows that warp 0 has consumed the previous phase of every stage, so
// the stage's parity is unambiguous for it: it then waits on the stage's own
// mbarrier directly and saves the hand-over.  The stage
// of a computed tile is free once its barrier has been passed, the stage of a
// copied tile once its store group has finished reading shared memory; warp 0
// keeps as many loads in flight as that rule allows (kS - 1 ahead of a computed
// tile, kS - 2 ahead of a copied one).
template <int kT, int kS>
__device__ __forceinline__ void transfer_body(const XferParams& p) {
  static_assert(kS >= 2, "a ring needs two stages; pure copies overlap loads with stores only from three stages on");
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kS];
  __shared__ uint32_t red[2][kT / 32];
  __shared__ __align__(8) uint64_t ready_bar;  // one phase per staged computed tile: warp 0 has seen its data (or gave up)
  __shared__ volatile int give_up;             // written by warp 0 before it arrives on ready_bar

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ready_addr = smem_addr(&ready_bar);
  if (threadIdx.x == 0) {
    give_up = 0;
    mbar_init(ready_addr, 1);
    for (int s = 0; s < kS; ++s) mbar_init(smem_addr(&full_bar[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Wait until every destination has announced this epoch (its engine is paused
  // and its parameters may be overwritten).  A CTA that gives up skips its tiles
  // but still drains and counts itself in below, so that the arrival counter is
  // back at zero when the launch ends.
  uint32_t my_abort = 0;
  if (p.n_ready) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = threadIdx.x; i < p.n_ready && !my_abort; i += blockDim.x) {
      const uint64_t* flag = p.ready_pad + p.ready_slots[i];
      while (ld_acquire_sys(flag) < p.epoch) {
        if (globaltimer_ns() - t0 > p.timeout_ns) {
          if (atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_READY_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(p.ready_slots[i]);
          my_abort = 1;
          break;
        }
        __nanosleep(200);
      }
    }
    my_abort = __syncthreads_or(static_cast<int>(my_abort)) != 0;
  }

  // Which tiles this CTA owns: its plan entry, or an even contiguous share.
  const bool planned = p.cta_plan != nullptr;
  const uint32_t cs = planned ? p.chunk_shift : 0;
  const uint64_t cmask = (uint64_t{1} << cs) - 1;
  uint64_t t_begin, n = 0;
  uint32_t g_rank = 0, g_size = 1, chunk_off = 0;
  if (planned) {
    const CtaPlan plan = p.cta_plan[blockIdx.x];
    t_begin = plan.tile_begin;
    g_rank = plan.rank;
    g_size = plan.size;
    chunk_off = plan.chunk_off;
    const uint64_t range = plan.tile_end - plan.tile_begin;
    const uint64_t n_chunks = (range + cmask) >> cs;
    if (g_rank < n_chunks) {
      const uint64_t mine = (n_chunks - g_rank + g_size - 1) / g_size;
      n = mine << cs;
      if (g_rank + (mine - 1) * g_size == n_chunks - 1) n -= (n_chunks << cs) - range;  // the range's last chunk may be short
    }
  } else {
    t_begin = p.n_tiles * blockIdx.x / gridDim.x;
    n = p.n_tiles * (blockIdx.x + 1) / gridDim.x - t_begin;
  }
  if (my_abort) n = 0;
  // relative tile number of this CTA -> tile number in the table
  auto cursor_to = [&](Cursor& c, uint64_t j) -> uint64_t {
    const uint64_t chunk = (j >> cs) * g_size + g_rank;
    const uint64_t tile = t_begin + (chunk << cs) + (j & cmask);
    if (planned && (j & cmask) == 0) cursor_jump(c, p, chunk_off + chunk);
    cursor_advance_to(c, p, tile);
    return tile;
  };

  uint64_t next_load = 0;  // warp 0: tiles [0, next_load) have had their loads issued
  uint64_t waited = 0;     // warp 0: tiles [0, waited) have been seen complete (or were never staged)
  if (n > 0) {
    Cursor load_cur, use_cur;
    if (planned) cursor_jump(load_cur, p, chunk_off + g_rank);
    else cursor_seek(load_cur, p, t_begin);
    use_cur = load_cur;

    // Stage tile j (relative number) of this CTA.  Executed by warp 0.
    auto issue_load = [&](uint64_t j) {
      const uint64_t tile_no = cursor_to(load_cur, j);
      const XferDesc d = p.descs[load_cur.di];
      const uint32_t stage = static_cast<uint32_t>(j % kS);
      const uint32_t bar = smem_addr(&full_bar[stage]);
      if (!wants_stage(d)) {
        if (lane == 0) mbar_arrive(bar);  // keeps the ring's phases in step
        return;
      }
      const Tile t = tile_of(d, tile_no - load_cur.begin);
      if (d.tensor_map) {
        // one tiled TMA load for the whole tile; rows and columns past the slab's
        // edge are zero-filled and still counted in the transaction bytes
        if (lane == 0) {
          const uint32_t box_bytes = d.tile_rows * stage_pitch(d);
          mbar_arrive_expect_tx(bar, box_bytes);
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                  smem_addr(smem + static_cast<size_t>(stage) * kStageBytes)),
              "l"(d.tensor_map), "r"(static_cast<int32_t>(t.col0)), "r"(static_cast<int32_t>(t.row0)), "r"(bar)
              : "memory");
        }
        return;
      }
      const uint32_t ses = dtype_size(d.src_dtype);
      const uint32_t pitch = stage_pitch(d);
      const uint32_t bytes = t.cols * ses;
      if (lane == 0) mbar_arrive_expect_tx(bar, bytes * t.rows);
      __syncwarp();
      const unsigned char* src = reinterpret_cast<const unsigned char*>(d.src) + t.col0 * ses;
      const uint32_t base = smem_addr(smem + static_cast<size_t>(stage) * kStageBytes);
      for (uint32_t r = lane; r < t.rows; r += 32) bulk_load(base + r * pitch, src + src_row_offset(d, t.row0 + r), bytes, bar);
    };

    bool prev_copy = false;  // warp 0: was the previous tile a pure copy?
    uint32_t n_computed = 0; // selects the half of `red` (two consecutive computed tiles never share one)
    uint32_t n_staged = 0;   // staged computed tiles so far: the phase of `ready_bar`
    uint64_t last_barrier = ~uint64_t{0} >> 1;  // the newest tile at whose barrier all warps met (none yet: far away)
    XferDesc d;              // descriptor of the tile in use
    uint32_t d_index = 0xFFFFFFFFu;
    for (uint64_t i = 0; i < n; ++i) {
      const uint64_t tile_no = cursor_to(use_cur, i);
      if (use_cur.di != d_index) {  // most tiles continue the previous tile's slab
        d = p.descs[use_cur.di];
        d_index = use_cur.di;
      }
      const Tile t = tile_of(d, tile_no - use_cur.begin);
      const uint32_t stage = static_cast<uint32_t>(i % kS);
      const uint32_t parity = static_cast<uint32_t>((i / kS) & 1);
      const uint32_t bar = smem_addr(&full_bar[stage]);
      unsigned char* stage_ptr = smem + static_cast<size_t>(stage) * kStageBytes;
      const bool staged = wants_stage(d);
      const bool is_copy = d.op == OP_COPY && staged;
      // a quantised tile that leaves through its stage keeps the stage busy like a copy does
      const bool out_bulk = d.op == OP_FP8_BLOCK && fp8_leaves_through_stage(d, t);

      if (warp == 0 && !my_abort) {
        // Of the store groups committed so far (one per tile) only the most recent
        // may still be reading shared memory: every stage before tile i - 1 is
        // free, and the one of tile i - 1 too unless that tile was a pure copy.
        bulk_wait_read_1();
        __syncwarp();
        const uint64_t limit = i + kS - (prev_copy ? 1 : 0);
        while (next_load < limit && next_load < n) issue_load(next_load++);
      }
      prev_copy = is_copy || out_bulk;

      if (is_copy) {
        if (warp == 0 && !my_abort) {
          const bool arrived = mbar_wait_bounded(bar, parity, p.timeout_ns);
          if (__any_sync(0xffffffffu, !arrived)) {
            if (lane == 0 && atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_LOAD_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(use_cur.di);
            my_abort = 1;  // warp 0 stops moving data; it keeps meeting the other warps at their barriers
          } else {
            waited = i + 1;
            const uint32_t pitch = stage_pitch(d);
            const uint32_t bytes = t.cols;  // OP_COPY counts bytes
            unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst) + t.row0 * d.dst_stride + t.col0;
            const uint32_t base = smem_addr(stage_ptr);
            for (uint32_t r = lane; r < t.rows; r += 32) bulk_store(dst + static_cast<int64_t>(r) * d.dst_stride, base + r * pitch, bytes);
            bulk_commit();
          }
        }
        continue;  // other warps have nothing to do for pure copies
      }

      if (staged) {
        const uint32_t ready_parity = n_staged & 1;
        ++n_staged;
        // Is the previous phase of this stage's mbarrier known to be over?  Yes in the ring's first
        // round, and when this thread met warp 0 at a computed tile's barrier less than a round ago
        // (warp 0 had consumed every earlier tile by then).
        const bool direct = i < kS || i - last_barrier < kS;
        if (warp == 0) {
          // every lane observes the completed phase itself; lane 0 then hands the
          // observation on to the other warps (arrive releases, their wait acquires)
          if (!my_abort) {
            const bool arrived = mbar_wait_bounded(bar, parity, p.timeout_ns);
            if (__any_sync(0xffffffffu, !arrived)) {
              if (lane == 0 && atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_LOAD_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(use_cur.di);
              my_abort = 1;
            } else {
              waited = i + 1;
            }
          }
          if (lane == 0) {
            if (my_abort) give_up = 1;
            mbar_arrive(ready_addr);
          }
        } else if (!my_abort) {
          const bool arrived = direct ? mbar_wait_bounded(bar, parity, 2 * p.timeout_ns) : mbar_wait_bounded(ready_addr, ready_parity, 2 * p.timeout_ns);
          if (!arrived) {  // warp 0 gives up first and says so
            if (atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_LOAD_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(use_cur.di);
            my_abort = 1;
          } else if (!direct && give_up) {
            my_abort = 1;
          }
        }
      } else if (warp == 0 && !my_abort) {
        waited = i + 1;
      }
      last_barrier = i;
      uint32_t* red_now = red[n_computed & 1];
      ++n_computed;
      bool stop;
      if (d.op == OP_FP8_BLOCK) {
        if (staged && d.src_dtype == DT_BF16) stop = tile_fp8_staged<kT, true>(d, t, stage_ptr, red_now, my_abort);
        else if (staged) stop = tile_fp8_staged<kT, false>(d, t, stage_ptr, red_now, my_abort);
        else stop = tile_fp8_generic(d, t, red_now, my_abort);
      } else if (staged) {
        stop = tile_elementwise_staged(d, t, stage_ptr, my_abort);
      } else {
        stop = tile_elementwise_global(d, t, my_abort);
      }
      if (stop) {  // the same for every thread of the CTA
        my_abort = 1;
        break;
      }
      if (warp == 0 && !my_abort) {
        if (out_bulk) {
          unsigned char* dst = reinterpret_cast<unsigned char*>(d.dst) + t.row0 * d.dst_stride + t.col0;
          const uint32_t base = smem_addr(stage_ptr);
          for (uint32_t r = lane; r < t.rows; r += 32) bulk_store(dst + static_cast<int64_t>(r) * d.dst_stride, base + r * kFp8Block, t.cols);
        }
        bulk_commit();  // one group per tile, empty unless the tile left through its stage
      }
    }
  }

  // Drain: nothing of this CTA may still be in flight when it returns, and its
  // writes must be visible system-wide before it counts itself in.
  if (warp == 0) {
    if (my_abort && lane == 0) {
      // loads that were issued but never consumed still write into this CTA's
      // shared memory: give them one more deadline, in issue order
      for (uint64_t j = waited; j < next_load; ++j)
        if (!mbar_wait_bounded(smem_addr(&full_bar[j % kS]), static_cast<uint32_t>((j / kS) & 1), p.timeout_ns)) break;
    }
    __syncwarp();
    bulk_wait_all();
    fence_proxy_async();
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(p.cta_counter, 1u) + 1u;
    if (arrived == gridDim.x) {
      __threadfence_system();
      const bool ok = *reinterpret_cast<volatile int32_t*>(p.status) == ST_OK;
      // A failed launch raises no flag: receivers time out and report instead of
      // consuming a partial update.
      if (ok)
        for (uint32_t i = 0; i < p.n_done; ++i) st_release_sys(p.done_flags[i], p.epoch);
      *p.cta_counter = 0;  // ready for the next launch on this stream
    }
  }
}

// One CTA of 512 threads per SM with a 6-stage ring: the variant for tables of
// plain copies, where one warp moves the data and depth matters.
__global__ void __launch_bounds__(kThreads, 1) fused_transfer_kernel(const __grid_constant__ XferParams p) {
  transfer_body<kThreads, kStages>(p);
}

// Two CTAs of 256 threads per SM with a 3-stage ring each: the variant for
// tables dominated by tiles that every warp works on (block quantisation,
// casts) and for strided copies of short runs.  What one CTA cannot overlap
// (a tile's barrier, the maximum search before the first store, the issue of
// many small row copies) a second resident CTA fills with another tile.
constexpr int kThreadsX2 = 256;
constexpr int kStagesX2 = 3;
__global__ void __launch_bounds__(kThreadsX2, 2) fused_transfer_kernel_x2(const __grid_constant__ XferParams p) {
  transfer_body<kThreadsX2, kStagesX2>(p);
}

// Three CTAs of 256 threads per SM with a 2-stage ring each: the variant for
// tables that are almost only quantised blocks.  A computed tile frees its stage
// at its barrier, so two stages still keep one load in flight per CTA, and the
// third resident CTA hides more of each tile's latency.  Pure copies are correct
// in this shape but do not overlap their loads with their stores.
constexpr int kThreadsX3 = 256;
constexpr int kStagesX3 = 2;
__global__ void __launch_bounds__(kThreadsX3, 3) fused_transfer_kernel_x3(const __grid_constant__ XferParams p) {
  transfer_body<kThreadsX3, kStagesX3>(p);
}

// ---------------------------------------------------------------- the lean block-fp8 kernel
// Tables of nothing but quantised blocks fetched by tiled TMA loads (the expert
// weights of a block-fp8 serving layout: nine tenths of its bytes) do not need
// the general kernel's machinery, whose registers hold it at two CTAs per SM.
// This kernel keeps the table walk out of the threads that compute: a producer
// warp walks the CTA's tiles, and for each one issues the TMA load and leaves a
// small record (where the block goes, its extent, where its scale goes) beside
// the stage; eight consumer warps wait for the stage's mbarrier, read the
// record, quantise from registers and store.  A consumed stage is handed back
// through an "empty" mbarrier.  72 registers, three CTAs per SM, two 32 KiB stages
// each.  Same plans, same flags, same status words and the same self-resetting
// arrival counter as the general kernel; the host launches it on the part of a
// table that qualifies and the general kernel on the rest.
constexpr int kLeanConsumers = 256;
constexpr int kLeanThreads = kLeanConsumers + 32;
constexpr int kLeanStages = 2;

struct alignas(16) Fp8Rec {
  uint64_t dst;         // first byte of the block in the destination
  int64_t dst_stride;   // bytes
  uint64_t scale_addr;  // where the block's scale goes
  uint32_t rows;        // rows of the block that exist
  uint32_t chunks;      // 16-byte source chunks per row that exist (8 values each)
  uint32_t flags;       // XferFlags of the descriptor
  uint32_t src_bf16;    // 1: bf16 source, 0: fp16
};

// CTA-wide OR over the consumer threads only (named barrier 1).
__device__ __forceinline__ bool consumers_or(bool mine) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(mine)), "r"(kLeanConsumers)
      : "memory");
  return out != 0;
}

__global__ void __launch_bounds__(kLeanThreads, 3) fp8_table_kernel(const __grid_constant__ XferParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kLeanStages];
  __shared__ __align__(8) uint64_t empty_bar[kLeanStages];
  __shared__ Fp8Rec recs[kLeanStages];
  __shared__ uint32_t red[2][kLeanConsumers / 32];

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kLeanStages; ++s) {
      mbar_init(smem_addr(&full_bar[s]), 1);
      mbar_init(smem_addr(&empty_bar[s]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // wait until every destination has announced this epoch (as in the general kernel)
  uint32_t my_abort = 0;
  if (p.n_ready) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = threadIdx.x; i < p.n_ready && !my_abort; i += blockDim.x) {
      const uint64_t* flag = p.ready_pad + p.ready_slots[i];
      while (ld_acquire_sys(flag) < p.epoch) {
        if (globaltimer_ns() - t0 > p.timeout_ns) {
          if (atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_READY_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(p.ready_slots[i]);
          my_abort = 1;
          break;
        }
        __nanosleep(200);
      }
    }
    my_abort = __syncthreads_or(static_cast<int>(my_abort)) != 0;
  }

  // this CTA's tiles: its plan entry, or an even contiguous share
  const bool planned = p.cta_plan != nullptr;
  const uint32_t cs = planned ? p.chunk_shift : 0;
  const uint64_t cmask = (uint64_t{1} << cs) - 1;
  uint64_t t_begin, n = 0;
  uint32_t g_rank = 0, g_size = 1, chunk_off = 0;
  if (planned) {
    const CtaPlan plan = p.cta_plan[blockIdx.x];
    t_begin = plan.tile_begin;
    g_rank = plan.rank;
    g_size = plan.size;
    chunk_off = plan.chunk_off;
    const uint64_t range = plan.tile_end - plan.tile_begin;
    const uint64_t n_chunks = (range + cmask) >> cs;
    if (g_rank < n_chunks) {
      const uint64_t mine = (n_chunks - g_rank + g_size - 1) / g_size;
      n = mine << cs;
      if (g_rank + (mine - 1) * g_size == n_chunks - 1) n -= (n_chunks << cs) - range;
    }
  } else {
    t_begin = p.n_tiles * blockIdx.x / gridDim.x;
    n = p.n_tiles * (blockIdx.x + 1) / gridDim.x - t_begin;
  }
  if (my_abort) n = 0;

  if (warp == kLeanConsumers / 32) {
    // ---- producer: one lane walks the table, issues the loads, writes the records
    if (lane == 0 && n > 0) {
      Cursor cur;
      if (planned) cursor_jump(cur, p, chunk_off + g_rank);
      else cursor_seek(cur, p, t_begin);
      uint64_t issued = 0;
      bool failed = false;
      for (uint64_t j = 0; j < n; ++j) {
        const uint32_t stage = static_cast<uint32_t>(j & 1);
        if (j >= kLeanStages) {  // the stage's previous block has been taken into registers by every consumer
          if (!mbar_wait_bounded(smem_addr(&empty_bar[stage]), static_cast<uint32_t>(((j >> 1) - 1) & 1), 2 * p.timeout_ns)) {
            failed = true;  // the consumers stopped (they have reported why)
            break;
          }
        }
        const uint64_t chunk = (j >> cs) * g_size + g_rank;
        const uint64_t tile = t_begin + (chunk << cs) + (j & cmask);
        if (planned && (j & cmask) == 0) cursor_jump(cur, p, chunk_off + chunk);
        cursor_advance_to(cur, p, tile);
        const XferDesc* d = &p.descs[cur.di];
        const uint32_t col_tiles = d->col_tiles;
        const uint32_t k = static_cast<uint32_t>(tile - cur.begin);
        const uint32_t band = k / col_tiles, ct = k - band * col_tiles;
        const uint64_t row0 = static_cast<uint64_t>(band) * kFp8Block, col0 = static_cast<uint64_t>(ct) * kFp8Block;
        const uint64_t rows_left = d->rows - row0, cols_left = d->row_elems - col0;
        Fp8Rec& rec = recs[stage];
        rec.dst = d->dst + row0 * d->dst_stride + col0;
        rec.dst_stride = d->dst_stride;
        rec.scale_addr = d->aux_ptr + (static_cast<int64_t>(band) * d->aux_stride + ct) * 4;
        rec.rows = rows_left < kFp8Block ? static_cast<uint32_t>(rows_left) : kFp8Block;
        rec.chunks = (cols_left < kFp8Block ? static_cast<uint32_t>(cols_left) : kFp8Block) >> 3;
        rec.flags = d->flags;
        rec.src_bf16 = d->src_dtype == DT_BF16;
        const uint32_t bar = smem_addr(&full_bar[stage]);
        mbar_arrive_expect_tx(bar, kStageBytes);  // releases the record; the whole 128 x 128 box counts, zero-filled past the slab's edge
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                smem_addr(smem + static_cast<size_t>(stage) * kStageBytes)),
            "l"(d->tensor_map), "r"(static_cast<int32_t>(col0)), "r"(static_cast<int32_t>(row0)), "r"(bar)
            : "memory");
        issued = j + 1;
      }
      if (failed || my_abort) {
        // nothing of this CTA may be in flight when it returns: the last loads issued get one more deadline
        for (uint64_t j = issued > kLeanStages ? issued - kLeanStages : 0; j < issued; ++j)
          if (!mbar_wait_bounded(smem_addr(&full_bar[j & 1]), static_cast<uint32_t>((j >> 1) & 1), p.timeout_ns)) break;
      }
    }
  } else {
    // ---- consumers
    const uint32_t chunk = threadIdx.x & 15u, row0 = threadIdx.x >> 4;
    constexpr int kPasses = (kFp8Block * kFp8Block * 2 / 16) / kLeanConsumers;  // 8 chunks per thread
    constexpr uint32_t kRowStep = kLeanConsumers / 16;
    for (uint64_t i = 0; i < n; ++i) {
      const uint32_t stage = static_cast<uint32_t>(i & 1);
      const bool arrived = mbar_wait_bounded(smem_addr(&full_bar[stage]), static_cast<uint32_t>((i >> 1) & 1), p.timeout_ns);
      if (!arrived && atomicCAS(reinterpret_cast<int*>(p.status), ST_OK, ST_LOAD_TIMEOUT) == ST_OK) p.status[1] = static_cast<int>(i);
      const Fp8Rec rec = recs[stage];
      const unsigned char* stage_ptr = smem + static_cast<size_t>(stage) * kStageBytes;
      const bool col_ok = arrived && chunk < rec.chunks;
      uint4 raw[kPasses];
      uint32_t m = 0;
#pragma unroll
      for (int q = 0; q < kPasses; ++q) {
        const uint32_t row = row0 + q * kRowStep;
        raw[q] = (col_ok && row < rec.rows) ? *reinterpret_cast<const uint4*>(stage_ptr + row * 256u + chunk * 16u) : make_uint4(0, 0, 0, 0);
        m = amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(m, raw[q].x), raw[q].y), raw[q].z), raw[q].w);
      }
      m = __reduce_max_sync(0xffffffffu, max(m & 0xFFFFu, m >> 16));
      if (lane == 0) red[i & 1][warp] = m;
      if (consumers_or(!arrived)) break;  // the same verdict for every consumer
      if (threadIdx.x == 0) mbar_arrive(smem_addr(&empty_bar[stage]));  // every consumer holds its part in registers
      uint32_t all = red[i & 1][0];
#pragma unroll
      for (int w = 1; w < kLeanConsumers / 32; ++w) all = max(all, red[i & 1][w]);
      const float amax = rec.src_bf16 ? __uint_as_float(all << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(all)));
      const QuantScale qs = make_quant_scale(amax, (rec.flags & FLAG_UE8M0) != 0);
      if (threadIdx.x == 0) *reinterpret_cast<float*>(rec.scale_addr) = qs.s;
      unsigned char* dst = reinterpret_cast<unsigned char*>(rec.dst) + chunk * 8u;
      const bool vec = (rec.flags & FLAG_DST_VEC16) != 0;
#pragma unroll
      for (int q = 0; q < kPasses; ++q) {
        const uint32_t row = row0 + q * kRowStep;
        if (!col_ok || row >= rec.rows) continue;
        const uint2 out = rec.src_bf16 ? quant_chunk16<true>(raw[q], qs) : quant_chunk16<false>(raw[q], qs);
        unsigned char* o = dst + static_cast<int64_t>(row) * rec.dst_stride;
        if (vec) {
          *reinterpret_cast<uint2*>(o) = out;
        } else {
          const unsigned char* b = reinterpret_cast<const unsigned char*>(&out);
          for (int j = 0; j < 8; ++j) o[j] = b[j];
        }
      }
    }
  }

  // Drain: this CTA's writes must be visible system-wide before it counts itself in.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(p.cta_counter, 1u) + 1u;
    if (arrived == gridDim.x) {
      __threadfence_system();
      const bool ok = *reinterpret_cast<volatile int32_t*>(p.status) == ST_OK;
      if (ok)
        for (uint32_t i = 0; i < p.n_done; ++i) st_release_sys(p.done_flags[i], p.epoch);
      *p.cta_counter = 0;
    }
  }
}

// Receiver side: wait (bounded) until every listed sender has raised `epoch`.
__global__ void wait_flags_kernel(const uint64_t* pad, const uint32_t* slots, uint32_t n, uint64_t epoch, uint64_t timeout_ns,
                                  int32_t* status) {
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint64_t* flag = pad + slots[i];
    while (ld_acquire_sys(flag) < epoch) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (atomicCAS(reinterpret_cast<int*>(status), ST_OK, ST_FLAG_TIMEOUT) == ST_OK) {
          status[1] = static_cast<int>(slots[i]);
          status[2] = static_cast<int>(ld_acquire_sys(flag));
        }
        break;
      }
      __nanosleep(200);
    }
  }
}

// Raise flags at (possibly peer-mapped) addresses, after everything this
// stream has written so far.
__global__ void post_flags_kernel(uint64_t* const* addrs, uint32_t n, uint64_t epoch) {
  __threadfence_system();
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) st_release_sys(addrs[i], epoch);
}

}  // namespace awex

// ---------------------------------------------------------------- host launchers
extern "C" {

int awex_xfer_desc_size() { return static_cast<int>(sizeof(awex::XferDesc)); }
int awex_xfer_smem_bytes() { return awex::kStages * awex::kStageBytes; }
int awex_xfer_stage_bytes() { return awex::kStageBytes; }

// Returns a cudaError_t.  `variant` 0: one CTA of 512 threads per SM; 1: two
// CTAs of 256 threads per SM; 2: three CTAs of 256 threads per SM; 3: the lean
// block-fp8 kernel (every descriptor must be a staged OP_FP8_BLOCK slab of a
// 2-byte type with a tensor map; the caller checks).  `grid` == 0 fills the device for the variant.
// With `cta_plan` (one CtaPlan per CTA, plus `chunk_desc`) `grid` is the number
// of plan entries and is used as given.
int awex_launch_fused_transfer(const void* descs, uint32_t n_desc, uint64_t n_tiles, uint64_t epoch, uint64_t timeout_ns,
                               const void* ready_pad, const void* ready_slots, uint32_t n_ready, const void* done_flags,
                               uint32_t n_done, void* cta_counter, void* status, int grid, void* stream,
                               const void* chunk_desc, uint32_t chunk_shift, uint32_t variant, const void* cta_plan) {
  // the shared-memory attribute is set once per (variant, device)
  static std::atomic<uint64_t> configured[4];
  if (variant > 3) return cudaErrorInvalidValue;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  const int stages = variant == 0 ? awex::kStages : variant == 1 ? awex::kStagesX2 : variant == 2 ? awex::kStagesX3 : awex::kLeanStages;
  const int smem = stages * awex::kStageBytes;
  const uint64_t bit = (dev >= 0 && dev < 64) ? (uint64_t{1} << dev) : 0;
  if (bit == 0 || !(configured[variant].load(std::memory_order_acquire) & bit)) {
    err = variant == 0   ? cudaFuncSetAttribute(awex::fused_transfer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
          : variant == 1 ? cudaFuncSetAttribute(awex::fused_transfer_kernel_x2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
          : variant == 2 ? cudaFuncSetAttribute(awex::fused_transfer_kernel_x3, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                         : cudaFuncSetAttribute(awex::fp8_table_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    configured[variant].fetch_or(bit, std::memory_order_release);
  }
  if (cta_plan != nullptr && (chunk_desc == nullptr || grid <= 0)) return cudaErrorInvalidValue;
  if (grid <= 0) {
    err = cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    grid *= variant == 3 ? 3 : static_cast<int>(variant) + 1;
  }
  if (cta_plan == nullptr && n_tiles > 0 && static_cast<uint64_t>(grid) > n_tiles) grid = static_cast<int>(n_tiles);
  if (grid < 1) grid = 1;
  awex::XferParams p;
  p.descs = static_cast<const awex::XferDesc*>(descs);
  p.n_desc = n_desc;
  p.n_tiles = n_desc ? n_tiles : 0;
  p.epoch = epoch;
  p.timeout_ns = timeout_ns;
  p.ready_pad = static_cast<const uint64_t*>(ready_pad);
  p.ready_slots = static_cast<const uint32_t*>(ready_slots);
  p.n_ready = n_ready;
  p.done_flags = static_cast<uint64_t* const*>(done_flags);
  p.n_done = n_done;
  p.cta_counter = static_cast<unsigned int*>(cta_counter);
  p.status = static_cast<int32_t*>(status);
  p.cta_plan = static_cast<const awex::CtaPlan*>(cta_plan);
  p.chunk_desc = static_cast<const uint32_t*>(chunk_desc);
  p.chunk_shift = cta_plan ? chunk_shift : 0;
  if (variant == 3)
    awex::fp8_table_kernel<<<grid, awex::kLeanThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  else if (variant == 2)
    awex::fused_transfer_kernel_x3<<<grid, awex::kThreadsX3, smem, static_cast<cudaStream_t>(stream)>>>(p);
  else if (variant == 1)
    awex::fused_transfer_kernel_x2<<<grid, awex::kThreadsX2, smem, static_cast<cudaStream_t>(stream)>>>(p);
  else
    awex::fused_transfer_kernel<<<grid, awex::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError();
}

int awex_launch_wait_flags(const void* pad, const void* slots, uint32_t n, uint64_t epoch, uint64_t timeout_ns, void* status,
                           void* stream) {
  if (n == 0) return cudaSuccess;
  awex::wait_flags_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint64_t*>(pad), static_cast<const uint32_t*>(slots), n, epoch, timeout_ns, static_cast<int32_t*>(status));
  return cudaGetLastError();
}

int awex_launch_post_flags(const void* addrs, uint32_t n, uint64_t epoch, void* stream) {
  if (n == 0) return cudaSuccess;
  awex::post_flags_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t* const*>(addrs), n, epoch);
  return cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------- allocation-free launch
// See awex_no_alloc.h for who calls this and under which rules.
#include <cstdio>
#include <mutex>

#include "awex_no_alloc.h"

namespace awex {

// Scratch of the allocation-free launch: [0, 4) CTA arrival counter, [16, 32)
// status words, [256, ...) descriptor table.  In host code this name is only a
// handle for the runtime's symbol calls; its device address is looked up once
// per device below.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[AWEX_NO_ALLOC_SCRATCH_BYTES];

static_assert(AWEX_NO_ALLOC_HEADER_BYTES % alignof(XferDesc) == 0, "table must start aligned");
static_assert(sizeof(XferDesc) == 128, "scratch size is stated in 128-byte descriptors");

constexpr int kNoAllocMaxDevices = 64;
static unsigned char* g_no_alloc_ptr[kNoAllocMaxDevices] = {};
static std::mutex g_no_alloc_mutex;

static int no_alloc_fail(cudaError_t code, char* err, size_t cap, const char* what) {
  if (err != nullptr && cap > 0) std::snprintf(err, cap, "awex_fused_transfer_no_alloc: %s (%s)", what, cudaGetErrorString(code));
  return static_cast<int>(code);
}

// Structure of a caller-built table, checked on the host before anything is
// queued: every rule here is one whose violation would make the kernel compute a
// tile outside its slab, overrun a pipeline stage or break a bulk copy's
// alignment.  Returns nullptr or what is wrong; `bad` gets the descriptor index.
static const char* no_alloc_check_structure(const XferDesc* t, uint32_t n_desc, uint64_t n_tiles, uint32_t* bad) {
  uint64_t expect = 0;
  for (uint32_t i = 0; i < n_desc; ++i) {
    const XferDesc& d = t[i];
    *bad = i;
    if (d.op > OP_FP8_BLOCK || d.src_dtype > DT_FP8_E4M3 || d.dst_dtype > DT_FP8_E4M3) return "unknown op or dtype";
    if (d.rows == 0 || d.row_elems == 0) return "empty slab";
    if (d.tile_rows == 0 || d.tile_cols == 0 || d.col_tiles == 0) return "tile_rows, tile_cols and col_tiles must be non-zero";
    if (d.col_tiles != (d.row_elems + d.tile_cols - 1) / d.tile_cols) return "col_tiles does not match row_elems / tile_cols";
    if (d.tile_begin != expect) return i == 0 ? "tile_begin of the first descriptor must be 0" : "tile_begin must continue the running tile count";
    expect += static_cast<uint64_t>(d.col_tiles) * ((d.rows + d.tile_rows - 1) / d.tile_rows);
    if (d.src == 0 || d.dst == 0) return "null source or destination";
    const uint32_t ses = d.src_dtype == DT_F32 ? 4u : (d.src_dtype == DT_BF16 || d.src_dtype == DT_F16) ? 2u : 1u;
    if (d.op == OP_COPY && (d.src_dtype != DT_BYTES || d.dst_dtype != DT_BYTES)) return "copies count bytes (dtype 0 on both sides)";
    if (d.op != OP_COPY && (d.src_dtype == DT_BYTES || d.dst_dtype == DT_BYTES)) return "a computed slab needs element dtypes";
    if (d.flags & FLAG_BULK) {
      const uint64_t pitch = (static_cast<uint64_t>(d.tile_cols) * ses + 15u) & ~uint64_t{15};
      if ((d.src & 15u) || ((d.row_elems * ses) & 15u) || ((static_cast<uint64_t>(d.tile_cols) * ses) & 15u) ||
          (d.rows > 1 && d.row_table == 0 && (d.src_stride & 15)))
        return "bulk source rule (16-byte address, stride and size) violated";
      if (d.op == OP_COPY && ((d.dst & 15u) || (d.rows > 1 && (d.dst_stride & 15)))) return "bulk destination rule (16-byte address and stride) violated";
      if (static_cast<uint64_t>(d.tile_rows) * pitch > static_cast<uint64_t>(kStageBytes)) return "a tile exceeds one pipeline stage";
      if (d.op == OP_FP8_BLOCK && ses != 2u) return "staged block quantisation needs a 2-byte source";
    } else if (d.tensor_map != 0) {
      return "a tensor map needs the bulk flag";
    }
    if (d.op == OP_FP8_BLOCK) {
      if (d.tile_rows != kFp8Block || d.tile_cols != kFp8Block) return "fp8 tiles must be 128 x 128";
      if (d.dst_dtype != DT_FP8_E4M3 || d.aux_ptr == 0 || (d.aux_ptr & 3u)) return "fp8 slab without an e4m3 destination or a float-aligned scale address";
    }
  }
  *bad = n_desc;
  if (expect != n_tiles) return "n_tiles does not match the table";
  return nullptr;
}

// Is `addr` memory a kernel on the current device can touch?  (Asks the driver
// about the pointer; allocates nothing.)  0 is accepted when `optional`.
static bool no_alloc_device_pointer(uint64_t addr, bool optional) {
  if (addr == 0) return optional;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, reinterpret_cast<const void*>(addr)) != cudaSuccess) {
    cudaGetLastError();  // not a pointer the runtime knows: leave no sticky error behind
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

}  // namespace awex

extern "C" int awex_fused_transfer_no_alloc(const void* host_descs, uint32_t n_desc, uint64_t n_tiles, uint64_t timeout_ns,
                                            int grid, void* stream, int32_t* status_out, char* err, size_t err_cap) {
  using namespace awex;
  if (err != nullptr && err_cap > 0) err[0] = '\0';
  if (n_desc > AWEX_NO_ALLOC_MAX_DESCS) {
    if (err != nullptr && err_cap > 0)
      std::snprintf(err, err_cap,
                    "awex_fused_transfer_no_alloc: %u descriptors exceed the built-in scratch of %u descriptors; split the table",
                    n_desc, AWEX_NO_ALLOC_MAX_DESCS);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  if (n_desc > 0 && host_descs == nullptr) return no_alloc_fail(cudaErrorInvalidValue, err, err_cap, "null descriptor table");
  const XferDesc* table = static_cast<const XferDesc*>(host_descs);
  if (n_desc > 0 && n_tiles > 0) {
    // The table is in host memory: prove before anything is queued that the kernel
    // will stay inside what it describes.
    uint32_t bad = 0;
    if (const char* what = no_alloc_check_structure(table, n_desc, n_tiles, &bad)) {
      if (err != nullptr && err_cap > 0) std::snprintf(err, err_cap, "awex_fused_transfer_no_alloc: descriptor %u: %s", bad, what);
      return static_cast<int>(cudaErrorInvalidValue);
    }
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "cudaGetDevice");
  if (dev < 0 || dev >= kNoAllocMaxDevices) return no_alloc_fail(cudaErrorInvalidDevice, err, err_cap, "device index beyond the per-device table");
  const int smem = kStages * kStageBytes;
  unsigned char* scratch = nullptr;
  {
    // once per device, with that device current
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
      if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "cudaGetSymbolAddress of the scratch array");
      e = cudaFuncSetAttribute(fused_transfer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "cudaFuncSetAttribute");
      g_no_alloc_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    scratch = g_no_alloc_ptr[dev];
  }
  if (n_desc > 0 && n_tiles > 0) {
    // Addresses the kernel dereferences must be device memory.  A table straight
    // from an encoder still holds row-table indices and no tensor-map addresses;
    // both are only meaningful once they point into device memory.
    for (uint32_t i = 0; i < n_desc; ++i) {
      const XferDesc& d = table[i];
      const char* what = nullptr;
      if (!no_alloc_device_pointer(d.row_table, true)) what = "row_table is neither 0 nor a device address";
      else if (!no_alloc_device_pointer(d.tensor_map, true)) what = "tensor_map is neither 0 nor a device address";
      else if (!no_alloc_device_pointer(d.src, false)) what = "src is not a device address";
      else if (!no_alloc_device_pointer(d.dst, false)) what = "dst is not a device address";
      else if (d.op == OP_FP8_BLOCK && !no_alloc_device_pointer(d.aux_ptr, false)) what = "the scale address is not a device address";
      if (what != nullptr) {
        if (err != nullptr && err_cap > 0) std::snprintf(err, err_cap, "awex_fused_transfer_no_alloc: descriptor %u: %s", i, what);
        return static_cast<int>(cudaErrorInvalidValue);
      }
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps the previous call's contents: counter and status start at zero.
  e = cudaMemsetAsync(scratch, 0, AWEX_NO_ALLOC_HEADER_BYTES, s);
  if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "clearing the scratch header");
  int32_t* status = reinterpret_cast<int32_t*>(scratch + 16);
  if (n_desc > 0 && n_tiles > 0) {
    e = cudaMemcpyAsync(scratch + AWEX_NO_ALLOC_HEADER_BYTES, host_descs, static_cast<size_t>(n_desc) * sizeof(XferDesc),
                        cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "copying the descriptor table");
    if (grid <= 0) {
      e = cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "cudaDeviceGetAttribute");
    }
    if (static_cast<uint64_t>(grid) > n_tiles) grid = static_cast<int>(n_tiles);
    if (grid < 1) grid = 1;
    XferParams p;
    p.descs = reinterpret_cast<const XferDesc*>(scratch + AWEX_NO_ALLOC_HEADER_BYTES);
    p.n_desc = n_desc;
    p.n_tiles = n_tiles;
    p.epoch = 0;
    p.timeout_ns = timeout_ns;
    p.ready_pad = nullptr;
    p.ready_slots = nullptr;
    p.n_ready = 0;
    p.done_flags = nullptr;
    p.n_done = 0;
    p.cta_counter = reinterpret_cast<unsigned int*>(scratch);
    p.status = status;
    p.cta_plan = nullptr;  // contiguous tile ranges
    p.chunk_desc = nullptr;
    p.chunk_shift = 0;
    fused_transfer_kernel<<<grid, kThreads, smem, s>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "kernel launch");
  }
  if (status_out != nullptr) {
    e = cudaMemcpyAsync(status_out, status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "reading the status words");
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return no_alloc_fail(e, err, err_cap, "cudaStreamSynchronize");
  }
  return static_cast<int>(cudaSuccess);
}
