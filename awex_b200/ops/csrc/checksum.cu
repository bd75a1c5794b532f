// Position-sensitive 64-bit checksums of many (possibly strided) tensors in one
// launch, plus a NaN count per tensor.
//
// A tensor is seen as `rows` rows of `row_bytes` bytes, `stride` bytes apart.
// Each row is cut into 8-byte words (the last one zero-padded); word j of row r
// has index i = r * words_per_row + j.  The checksum is
//     sum_i mix(word_i) * K_i   (mod 2^64),   mix(w) = w ^ (w >> 32),   K_i = GOLDEN * (2 i + 1)
// mix is a bijection and every K_i is odd, so a change confined to one word
// always changes the sum.  Exchanging two different words at i != j changes it
// by (m_i - m_j) * 2 (j - i) * GOLDEN with m = mix(w); that vanishes modulo 2^64
// only when the powers of two dividing (m_i - m_j) and (j - i) add up to 63 or
// more.  Folding the high half into the low half keeps a difference in the top
// bits (the sign of a word's last element) from being such a case: words that
// differ only in bit 63 differ in bit 31 after mixing.  The check is a structured
// hash, not a proof: it catches swapped rows, shifted shards and missing writes,
// and two different tensors collide only by accident.  The sum is
// order-independent, so CTAs combine partial sums with one atomic add each, and
// it costs one 64-bit multiply-add per word, which keeps the kernel on the
// memory roofline.
//
// Used for weight validation: the reference copies every parameter to the host
// and compares there (awex/reader/weights_reader.py:436-587); here only 16
// bytes per parameter leave the GPU.

#include <cuda_runtime.h>

#include <cstdint>

namespace awex {

struct alignas(16) SumDesc {
  uint64_t ptr;
  uint64_t rows;
  uint64_t row_bytes;
  int64_t stride;
  uint64_t chunk_begin;     // number of this tensor's first chunk
  uint32_t rows_per_chunk;  // >= 1 when a chunk holds whole rows
  uint32_t chunks_per_row;  // >= 1 when a row is cut into several chunks
  uint32_t out_index;
  uint32_t dtype;           // 0 opaque, 1 bf16, 2 f16, 3 f32, 4 fp8 e4m3
};
static_assert(sizeof(SumDesc) == 56 + 8, "layout shared with the Python encoder");

// A chunk is what one CTA sums between two lookups in the descriptor table and
// two atomics: large enough (128 KiB) that those fixed costs stay small.
constexpr uint32_t kChunkWords = 16384;
constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

__device__ __forceinline__ uint64_t key_of(uint64_t i) { return kGolden * (2 * i + 1); }
__device__ __forceinline__ uint64_t mix(uint64_t w) { return w ^ (w >> 32); }
// 16 bytes that are read once: keep them out of L1
__device__ __forceinline__ ulonglong2 load_stream16(const unsigned char* p) {
  ulonglong2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p));
  return v;
}

// NaNs in a full 8-byte word, two SIMD compares per word.
__device__ __forceinline__ uint32_t count_nans_full(uint64_t w, uint32_t dtype) {
  const uint32_t lo = static_cast<uint32_t>(w), hi = static_cast<uint32_t>(w >> 32);
  if (dtype == 1) return (__popc(__vcmpgtu2(lo & 0x7FFF7FFFu, 0x7F807F80u)) + __popc(__vcmpgtu2(hi & 0x7FFF7FFFu, 0x7F807F80u))) >> 4;
  if (dtype == 2) return (__popc(__vcmpgtu2(lo & 0x7FFF7FFFu, 0x7C007C00u)) + __popc(__vcmpgtu2(hi & 0x7FFF7FFFu, 0x7C007C00u))) >> 4;
  if (dtype == 3) return ((lo & 0x7FFFFFFFu) > 0x7F800000u) + ((hi & 0x7FFFFFFFu) > 0x7F800000u);
  if (dtype == 4) return (__popc(__vcmpeq4(lo & 0x7F7F7F7Fu, 0x7F7F7F7Fu)) + __popc(__vcmpeq4(hi & 0x7F7F7F7Fu, 0x7F7F7F7Fu))) >> 3;
  return 0;
}

__device__ __forceinline__ uint32_t count_nans(uint64_t w, uint32_t dtype, uint32_t valid_bytes) {
  if (valid_bytes == 8) return count_nans_full(w, dtype);
  uint32_t n = 0;
  if (dtype == 1 || dtype == 2) {
    const uint32_t emask = dtype == 1 ? 0x7F80u : 0x7C00u, mmask = dtype == 1 ? 0x007Fu : 0x03FFu;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t h = static_cast<uint32_t>(w >> (16 * k)) & 0xFFFFu;
      n += (2u * k < valid_bytes) && ((h & emask) == emask) && (h & mmask);
    }
  } else if (dtype == 3) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint32_t f = static_cast<uint32_t>(w >> (32 * k));
      n += (4u * k < valid_bytes) && ((f & 0x7F800000u) == 0x7F800000u) && (f & 0x007FFFFFu);
    }
  } else if (dtype == 4) {
#pragma unroll
    for (int k = 0; k < 8; ++k) n += (static_cast<uint32_t>(k) < valid_bytes) && ((static_cast<uint32_t>(w >> (8 * k)) & 0x7Fu) == 0x7Fu);
  }
  return n;
}

__device__ __forceinline__ uint64_t load_word(const unsigned char* row, uint64_t j, uint64_t row_bytes, bool aligned, uint32_t* valid) {
  const uint64_t off = j * 8;
  const uint64_t left = row_bytes - off;
  *valid = left >= 8 ? 8u : static_cast<uint32_t>(left);
  if (aligned && left >= 8) return __ldg(reinterpret_cast<const unsigned long long*>(row + off));
  uint64_t w = 0;
  for (uint32_t b = 0; b < *valid; ++b) w |= static_cast<uint64_t>(row[off + b]) << (8 * b);
  return w;
}

__global__ void __launch_bounds__(256) checksum_kernel(const SumDesc* descs, uint32_t n_desc, uint64_t n_chunks,
                                                       unsigned long long* sums, unsigned long long* nans) {
  __shared__ unsigned long long red_sum[8];
  __shared__ unsigned int red_nan[8];
  for (uint64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    uint32_t lo = 0, hi = n_desc - 1;
    while (lo < hi) {
      uint32_t mid = (lo + hi + 1) >> 1;
      if (descs[mid].chunk_begin <= chunk) lo = mid; else hi = mid - 1;
    }
    const SumDesc d = descs[lo];
    const uint64_t k = chunk - d.chunk_begin;
    const uint64_t wpr = (d.row_bytes + 7) / 8;
    const unsigned char* base = reinterpret_cast<const unsigned char*>(d.ptr);
    const bool aligned = ((d.ptr | static_cast<uint64_t>(d.stride)) & 7) == 0;
    uint64_t acc = 0;
    uint32_t nan_acc = 0;
    if (d.chunks_per_row >= 1 && d.rows_per_chunk <= 1) {  // (part of) one row
      const uint64_t r = k / d.chunks_per_row, part = k % d.chunks_per_row;
      const uint64_t j0 = part * kChunkWords;
      const uint64_t j1 = min(j0 + static_cast<uint64_t>(kChunkWords), wpr);
      const unsigned char* row = base + static_cast<int64_t>(r) * d.stride;
      const uint64_t full_words = d.row_bytes / 8;  // words that need no padding
      const uint64_t jv1 = min(j1, full_words) & ~1ull;
      const uint64_t idx0 = r * wpr;
      uint64_t j = j0;
      if (aligned && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
        // two words per 16-byte load, kUnroll independent loads in flight per thread
        constexpr int kUnroll = 8;
        const uint64_t step = 2ull * blockDim.x;
        const uint64_t key_step = kGolden * 2 * step;
        j = j0 + 2ull * threadIdx.x;
        uint64_t key = key_of(idx0 + j);
        for (; j + (kUnroll - 1) * step < jv1; j += kUnroll * step) {
          ulonglong2 v[kUnroll];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) v[u] = load_stream16(row + (j + u * step) * 8);
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            acc += mix(v[u].x) * key + mix(v[u].y) * (key + 2 * kGolden);
            nan_acc += count_nans_full(v[u].x, d.dtype) + count_nans_full(v[u].y, d.dtype);
            key += key_step;
          }
        }
        for (; j < jv1; j += step, key += key_step) {
          const ulonglong2 a = load_stream16(row + j * 8);
          acc += mix(a.x) * key + mix(a.y) * (key + 2 * kGolden);
          nan_acc += count_nans_full(a.x, d.dtype) + count_nans_full(a.y, d.dtype);
        }
        j = max(j0, jv1);
      }
      for (j += threadIdx.x; j < j1; j += blockDim.x) {
        uint32_t valid;
        uint64_t w = load_word(row, j, d.row_bytes, aligned, &valid);
        acc += mix(w) * key_of(idx0 + j);
        nan_acc += count_nans(w, d.dtype, valid);
      }
    } else {  // several whole (short) rows: one warp per row
      const uint64_t r0 = k * d.rows_per_chunk;
      const uint64_t r1 = min(r0 + static_cast<uint64_t>(d.rows_per_chunk), d.rows);
      for (uint64_t r = r0 + (threadIdx.x >> 5); r < r1; r += blockDim.x >> 5) {
        const unsigned char* row = base + static_cast<int64_t>(r) * d.stride;
        for (uint64_t j = threadIdx.x & 31; j < wpr; j += 32) {
          uint32_t valid;
          uint64_t w = load_word(row, j, d.row_bytes, aligned, &valid);
          acc += mix(w) * key_of(r * wpr + j);
          nan_acc += count_nans(w, d.dtype, valid);
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      acc += __shfl_xor_sync(0xffffffffu, acc, off);
      nan_acc += __shfl_xor_sync(0xffffffffu, nan_acc, off);
    }
    if ((threadIdx.x & 31) == 0) {
      red_sum[threadIdx.x >> 5] = acc;
      red_nan[threadIdx.x >> 5] = nan_acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long s = 0;
      unsigned int nn = 0;
      for (int w = 0; w < 8; ++w) {
        s += red_sum[w];
        nn += red_nan[w];
      }
      atomicAdd(&sums[d.out_index], s);
      if (nn) atomicAdd(&nans[d.out_index], static_cast<unsigned long long>(nn));
    }
    __syncthreads();
  }
}

}  // namespace awex

extern "C" {

int awex_sum_desc_size() { return static_cast<int>(sizeof(awex::SumDesc)); }
int awex_sum_chunk_words() { return static_cast<int>(awex::kChunkWords); }

// `sums` and `nans` (one u64 per output slot) must be zeroed by the caller.
int awex_launch_checksum(const void* descs, uint32_t n_desc, uint64_t n_chunks, void* sums, void* nans, int grid, void* stream) {
  if (n_desc == 0 || n_chunks == 0) return cudaSuccess;
  if (grid <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    grid = sms * 8;
  }
  if (static_cast<uint64_t>(grid) > n_chunks) grid = static_cast<int>(n_chunks);
  awex::checksum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const awex::SumDesc*>(descs), n_desc, n_chunks, static_cast<unsigned long long*>(sums),
      static_cast<unsigned long long*>(nans));
  return cudaGetLastError();
}

}  // extern "C"
