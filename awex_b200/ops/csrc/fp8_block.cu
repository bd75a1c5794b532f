// Stand-alone block-scaled fp8 (e4m3) quantisation and dequantisation for sm_100a.
//
// Contract (the plain-PyTorch statement is per_block_cast_to_fp8 in
// awex_b200/converter/weights_converter.py; reference: awex/converter/
// weights_converter.py:42-61): 128x128 blocks over a zero-padded view of a 2-D
// tensor, scale = max(amax, 1e-4) / 448 in fp32 (optionally rounded up to a power
// of two), q = e4m3(x / scale) with a true division.
//
// Quantisation: persistent CTAs, one 128x128 block per iteration.  The block is
// fetched with ONE tiled TMA load (cp.async.bulk.tensor.2d, completion on an
// mbarrier) into a double-buffered stage; out-of-range rows/columns of edge
// blocks are zero-filled by the TMA unit, which is exactly the reference's
// zero padding.  Threads read the stage as consecutive 16-byte chunks (no bank
// conflicts) twice: once for the block maximum (integer SIMD on magnitude bits),
// once to quantise (exact without a division per element, see fp8_math.cuh) and
// write e4m3 with coalesced 8-byte stores.  The reference spends ~10 ATen kernels and a padded
// temporary on the same math.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <type_traits>

#include "fp8_math.cuh"

namespace awex {

constexpr int kBlk = 128;
constexpr int kQThreads = 256;

__device__ __forceinline__ uint32_t q_smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }

// Bounded wait for one phase of an mbarrier (spin budget far beyond any real latency).
__device__ __forceinline__ bool q_wait(uint32_t bar, uint32_t parity) {
  uint32_t done = 0;
  for (uint32_t spin = 0; !done && spin <= (1u << 24); ++spin)
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
  return done != 0;
}

// status: int32[4]; code 2 = a TMA load did not complete within the spin budget
//
// One pass over each staged block: a thread keeps its 16-byte chunks in
// registers from the maximum search, the CTA agrees on the block maximum with
// one barrier (the reduction scratch alternates between two halves, so nothing
// else has to protect it), and the values are quantised from the registers.
// After that barrier nobody reads the stage, so the load of the block after
// next goes into it right away: two loads are in flight while a block is
// quantised.
template <typename T>
__global__ void __launch_bounds__(kQThreads, sizeof(T) == 4 ? 1 : 3)
fp8_block_quant_kernel(const __grid_constant__ CUtensorMap x_map, unsigned char* __restrict__ q, float* __restrict__ scales,
                       uint32_t rows, uint32_t cols, int64_t q_stride, int64_t scale_stride, uint32_t blocks_n,
                       uint32_t n_blocks, int ue8m0, int32_t* status) {
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t red[2][kQThreads / 32];
  constexpr uint32_t kStage = kBlk * kBlk * sizeof(T);
  constexpr int kChunkElems = 16 / sizeof(T);          // elements per 16-byte chunk
  constexpr int kChunksPerRow = kBlk / kChunkElems;    // 16 (2-byte types) or 32 (fp32)
  constexpr int kRowsPerPass = kQThreads / kChunksPerRow;
  constexpr int kPasses = kBlk / kRowsPerPass;
  const uint32_t tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < 2; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(q_smem_addr(&bars[s])), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](uint32_t blk, uint32_t stage) {  // thread 0 only
    const uint32_t bar = q_smem_addr(&bars[stage]);
    const int32_t x0 = static_cast<int32_t>((blk % blocks_n) * kBlk);  // element column: a multiple of 128, so 16-byte aligned
    const int32_t y0 = static_cast<int32_t>((blk / blocks_n) * kBlk);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kStage) : "memory");
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            q_smem_addr(stage_mem + stage * kStage)),
        "l"(reinterpret_cast<uint64_t>(&x_map)), "r"(x0), "r"(y0), "r"(bar)
        : "memory");
  };

  uint32_t it = 0;
  uint32_t issued = 0;  // thread 0: loads issued so far (block numbers blockIdx.x + k * gridDim.x)
  if (tid == 0)
    for (; issued < 2 && blockIdx.x + static_cast<uint64_t>(issued) * gridDim.x < n_blocks; ++issued)
      issue(blockIdx.x + issued * gridDim.x, issued);
  bool gave_up = false;
  for (uint32_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x, ++it) {
    const uint32_t stage = it & 1, parity = (it >> 1) & 1;
    // every thread observes the completed phase itself, which orders the staged bytes before its reads
    const bool arrived = q_wait(q_smem_addr(&bars[stage]), parity);
    if (!arrived && status && atomicCAS(status, 0, 2) == 0) status[1] = static_cast<int32_t>(blk);
    const unsigned char* stage_ptr = stage_mem + stage * kStage;
    const uint32_t chunk = tid % kChunksPerRow, row_in_pass = tid / kChunksPerRow;
    // the block's values, and their maximum as ordered magnitude bits (NaN sorts above infinity)
    uint4 raw[kPasses];
    uint32_t m = 0;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const uint32_t r = p * kRowsPerPass + row_in_pass;
      raw[p] = arrived ? *reinterpret_cast<const uint4*>(stage_ptr + (r * kChunksPerRow + chunk) * 16) : make_uint4(0, 0, 0, 0);
      if constexpr (sizeof(T) == 2) {
        m = amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(amax_bits_bf16x2(m, raw[p].x), raw[p].y), raw[p].z), raw[p].w);
      } else {
        m = max(max(m, raw[p].x & 0x7FFFFFFFu), max(raw[p].y & 0x7FFFFFFFu, max(raw[p].z & 0x7FFFFFFFu, raw[p].w & 0x7FFFFFFFu)));
      }
    }
    if constexpr (sizeof(T) == 2) m = max(m & 0xFFFFu, m >> 16);
    m = __reduce_max_sync(0xffffffffu, m);
    if ((tid & 31) == 0) red[it & 1][tid >> 5] = m;
    if (__syncthreads_or(arrived ? 0 : 1)) {  // the same verdict for every thread
      gave_up = true;
      break;
    }
    if (tid == 0) {
      const uint64_t after_next = blk + 2ull * gridDim.x;
      if (after_next < n_blocks) {
        issue(static_cast<uint32_t>(after_next), stage);  // everyone holds this stage's values in registers
        ++issued;
      }
    }
    uint32_t all = red[it & 1][0];
#pragma unroll
    for (int w = 1; w < kQThreads / 32; ++w) all = max(all, red[it & 1][w]);
    float amax;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) amax = __uint_as_float(all << 16);
    else if constexpr (std::is_same<T, __half>::value) amax = __half2float(__ushort_as_half(static_cast<unsigned short>(all)));
    else amax = __uint_as_float(all);
    const QuantScale qs = make_quant_scale(amax, ue8m0 != 0);
    const uint32_t brow = blk / blocks_n, bcol = blk % blocks_n;
    if (tid == 0) scales[static_cast<int64_t>(brow) * scale_stride + bcol] = qs.s;
    const uint32_t col0 = bcol * kBlk + chunk * kChunkElems;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const uint32_t r = brow * kBlk + p * kRowsPerPass + row_in_pass;
      if (r >= rows || col0 >= cols) continue;
      unsigned char* o = q + static_cast<int64_t>(r) * q_stride + col0;
      const bool whole = col0 + kChunkElems <= cols;
      if constexpr (sizeof(T) == 2) {
        const uint2 out = quant_chunk16<std::is_same<T, __nv_bfloat16>::value>(raw[p], qs);
        if (whole && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
          *reinterpret_cast<uint2*>(o) = out;
        } else {
          const unsigned char* b = reinterpret_cast<const unsigned char*>(&out);
          for (int j = 0; j < kChunkElems; ++j)
            if (col0 + j < cols) o[j] = b[j];
        }
      } else {
        const uint32_t out = quant_pair(__uint_as_float(raw[p].x), __uint_as_float(raw[p].y), qs) |
                             (quant_pair(__uint_as_float(raw[p].z), __uint_as_float(raw[p].w), qs) << 16);
        if (whole && (reinterpret_cast<uintptr_t>(o) & 3) == 0) {
          *reinterpret_cast<uint32_t*>(o) = out;
        } else {
          for (int j = 0; j < kChunkElems; ++j)
            if (col0 + j < cols) o[j] = static_cast<unsigned char>(out >> (8 * j));
        }
      }
    }
  }
  if (gave_up && tid == 0) {
    // loads that were issued but not consumed may still be writing into this
    // CTA's shared memory: one more bounded wait for each, oldest first
    for (uint32_t k = it; k < issued; ++k)
      if (!q_wait(q_smem_addr(&bars[k & 1]), (k >> 1) & 1)) break;
  }
}

// x = float(q) * scale(block); 16 fp8 values per thread and iteration.
template <typename T>
__global__ void __launch_bounds__(256) fp8_block_dequant_kernel(const unsigned char* __restrict__ q, const float* __restrict__ scales,
                                                                T* __restrict__ out, uint32_t rows, uint32_t cols, int64_t q_stride,
                                                                int64_t scale_stride, int64_t out_stride) {
  const uint32_t chunks_per_row = (cols + 15) / 16;
  const uint64_t total = static_cast<uint64_t>(rows) * chunks_per_row;
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint32_t r = static_cast<uint32_t>(i / chunks_per_row), c0 = static_cast<uint32_t>(i % chunks_per_row) * 16;
    const float s = scales[static_cast<int64_t>(r / kBlk) * scale_stride + c0 / kBlk];
    const unsigned char* src = q + static_cast<int64_t>(r) * q_stride + c0;
    T* dst = out + static_cast<int64_t>(r) * out_stride + c0;
    unsigned char b[16];
    const bool whole = c0 + 16 <= cols;
    if (whole && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      *reinterpret_cast<uint4*>(b) = __ldg(reinterpret_cast<const uint4*>(src));
    } else {
      for (int j = 0; j < 16; ++j) b[j] = (c0 + j < cols) ? src[j] : 0;
    }
    T vals[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __half_raw h = __nv_cvt_fp8_to_halfraw(b[j], __NV_E4M3);
      const float f = __half2float(*reinterpret_cast<__half*>(&h)) * s;
      if constexpr (sizeof(T) == 4) vals[j] = f;
      else if constexpr (std::is_same<T, __half>::value) vals[j] = __float2half_rn(f);
      else vals[j] = __float2bfloat16_rn(f);
    }
    if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int v = 0; v < static_cast<int>(sizeof(T)); ++v) reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(vals)[v];
    } else {
      for (int j = 0; j < 16; ++j)
        if (c0 + j < cols) dst[j] = vals[j];
    }
  }
}

// Exhaustive check of the division-free quotient used for 16-bit sources: every
// non-negative amax bit pattern of the type (one per blockIdx.x) against every
// value bit pattern of the type (threads stride over all 65536), for plain and
// power-of-two scales.  A value takes part when it can occur in a block with
// that maximum (|x| <= amax, or NaN / infinity, which make the scale non-finite
// and take the division anyway).  Counts the pairs whose e4m3 byte differs from
// the one the true division gives (must be none), and those whose fp32 quotient
// differs in its last bits (allowed: they never change the byte).
template <bool kBf16>
__global__ void fp8_quotient_check_kernel(unsigned long long* out) {
  const uint32_t amax_bits = blockIdx.x;  // 0 .. 0x7FFF
  const float amax = kBf16 ? __uint_as_float(amax_bits << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(amax_bits)));
  unsigned long long bad_bytes = 0, bad_quotients = 0, checked = 0;
  for (int ue8m0 = 0; ue8m0 < 2; ++ue8m0) {
    const QuantScale qs = make_quant_scale(amax, ue8m0 != 0);
    for (uint32_t xb = threadIdx.x; xb < 65536u; xb += blockDim.x) {
      const float x = kBf16 ? __uint_as_float(xb << 16) : __half2float(__ushort_as_half(static_cast<unsigned short>(xb)));
      if (!(fabsf(x) <= amax) && amax == amax && !isinf(amax)) continue;  // cannot occur in a block with this maximum
      const uint32_t want = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x, qs.s), 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFFu;
      // through the very function the kernels call, the value in each of the eight positions of a chunk in turn
      const uint32_t pos = xb & 7u;
      uint32_t words[4] = {0u, 0u, 0u, 0u};
      words[pos >> 1] = xb << (16 * (pos & 1u));
      const uint2 bytes = quant_chunk16<kBf16>(make_uint4(words[0], words[1], words[2], words[3]), qs);
      const uint32_t got = ((pos < 4 ? bytes.x : bytes.y) >> (8 * (pos & 3u))) & 0xFFu;
      ++checked;
      if (want != got) {
        ++bad_bytes;
        // remember one example: amax bits, value bits, scale kind, wanted and produced byte
        atomicCAS(&out[3], 0ull, 1ull | (static_cast<unsigned long long>(amax_bits) << 48) | (static_cast<unsigned long long>(xb) << 32) |
                                      (static_cast<unsigned long long>(ue8m0) << 24) | (want << 8) | got << 16);
      }
      if (qs.finite && __float_as_uint(quotient_corrected(x, qs)) != __float_as_uint(__fdiv_rn(x, qs.s))) ++bad_quotients;
    }
  }
  atomicAdd(&out[0], bad_bytes);
  atomicAdd(&out[1], bad_quotients);
  atomicAdd(&out[2], checked);
}

// scale[i] = the scale the quantisation kernels derive from a block maximum amax[i].
__global__ void fp8_scale_table_kernel(const float* __restrict__ amax, float* __restrict__ scale, uint32_t n, int ue8m0) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = make_quant_scale(amax[i], ue8m0 != 0).s;
}

}  // namespace awex

// ---------------------------------------------------------------- host launchers
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

template <typename T>
int launch_quant(const void* x, void* q, void* scales, uint64_t rows, uint64_t cols, int64_t x_stride, int64_t q_stride,
                 int64_t scale_stride, CUtensorMapDataType dt, int ue8m0, void* status, cudaStream_t stream) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return -1;
  // TMA rules: 16-byte aligned base, row pitch a multiple of 16 bytes
  if ((reinterpret_cast<uintptr_t>(x) & 15) || ((x_stride * sizeof(T)) & 15)) return -2;
  CUtensorMap map;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(x_stride) * sizeof(T)};
  const cuuint32_t box[2] = {awex::kBlk, awex::kBlk};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode(&map, dt, 2, const_cast<void*>(x), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
  const uint32_t blocks_m = static_cast<uint32_t>((rows + awex::kBlk - 1) / awex::kBlk);
  const uint32_t blocks_n = static_cast<uint32_t>((cols + awex::kBlk - 1) / awex::kBlk);
  const uint32_t n_blocks = blocks_m * blocks_n;
  if (n_blocks == 0) return cudaSuccess;
  const int smem = 2 * awex::kBlk * awex::kBlk * sizeof(T);
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  // the shared-memory attribute belongs to a (function, device) pair: one process may drive several GPUs
  static std::atomic<uint64_t> configured{0};
  const uint64_t bit = dev < 64 ? (uint64_t{1} << dev) : 0;
  if (!(configured.load(std::memory_order_acquire) & bit) || bit == 0) {
    e = cudaFuncSetAttribute(awex::fp8_block_quant_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured.fetch_or(bit, std::memory_order_release);
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int per_sm = sizeof(T) == 4 ? 1 : 3;  // 64 KiB (2-byte types) or 128 KiB (fp32) of stages per CTA
  uint32_t grid = static_cast<uint32_t>(sms * per_sm);
  if (grid > n_blocks) grid = n_blocks;
  awex::fp8_block_quant_kernel<T><<<grid, awex::kQThreads, smem, stream>>>(
      map, static_cast<unsigned char*>(q), static_cast<float*>(scales), static_cast<uint32_t>(rows), static_cast<uint32_t>(cols),
      q_stride, scale_stride, blocks_n, n_blocks, ue8m0, static_cast<int32_t*>(status));
  return cudaGetLastError();
}

template <typename T>
int launch_dequant(const void* q, const void* scales, void* out, uint64_t rows, uint64_t cols, int64_t q_stride, int64_t scale_stride,
                   int64_t out_stride, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const uint64_t work = rows * ((cols + 15) / 16);
  uint64_t grid = (work + 255) / 256;
  if (grid > static_cast<uint64_t>(sms) * 16) grid = static_cast<uint64_t>(sms) * 16;
  awex::fp8_block_dequant_kernel<T><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
      static_cast<const unsigned char*>(q), static_cast<const float*>(scales), static_cast<T*>(out), static_cast<uint32_t>(rows),
      static_cast<uint32_t>(cols), q_stride, scale_stride, out_stride);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

// Encode a 2-D tiled tensor map (no swizzle, zero fill) over a row-major slab.
// `elem_bytes` is 1, 2 or 4.  Returns 0 on success.
int awex_encode_tensor_map_2d(void* out_map128, int elem_bytes, uint64_t base, uint64_t cols, uint64_t rows,
                              uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return -1;
  if ((base & 15) || (row_pitch_bytes & 15) || box_cols > 256 || box_rows > 256) return -2;
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode(static_cast<CUtensorMap*>(out_map128), dt, 2, reinterpret_cast<void*>(base), dims, strides, box,
                      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

// dtype codes as in xfer_desc.h: 1 bf16, 2 f16, 3 f32.  Strides in elements.
// Returns 0, a cudaError_t, -1 (driver entry point missing) or -2 (input does
// not meet the TMA alignment rules; callers then use the fused transfer kernel).
int awex_launch_fp8_block_quant(const void* x, void* q, void* scales, uint64_t rows, uint64_t cols, int64_t x_stride,
                                int64_t q_stride, int64_t scale_stride, int src_dtype, int ue8m0, void* status, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (src_dtype) {
    case 1: return launch_quant<__nv_bfloat16>(x, q, scales, rows, cols, x_stride, q_stride, scale_stride, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ue8m0, status, s);
    case 2: return launch_quant<__half>(x, q, scales, rows, cols, x_stride, q_stride, scale_stride, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, ue8m0, status, s);
    case 3: return launch_quant<float>(x, q, scales, rows, cols, x_stride, q_stride, scale_stride, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, ue8m0, status, s);
    default: return -3;
  }
}

// out[4] (zeroed by the caller): e4m3 bytes that differ from the true division, fp32 quotients
// that differ, pairs checked, one packed example of a differing byte.  src_dtype 1: bf16, 2: fp16.
int awex_launch_fp8_quotient_check(int src_dtype, void* out, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (src_dtype == 1) awex::fp8_quotient_check_kernel<true><<<0x8000, 256, 0, s>>>(static_cast<unsigned long long*>(out));
  else if (src_dtype == 2) awex::fp8_quotient_check_kernel<false><<<0x8000, 256, 0, s>>>(static_cast<unsigned long long*>(out));
  else return -3;
  return cudaGetLastError();
}

// The scale rule alone, for exhaustive checks of its rounding: scale[i] from amax[i].
int awex_launch_fp8_scale_table(const void* amax, void* scale, uint32_t n, int ue8m0, void* stream) {
  if (n == 0) return cudaSuccess;
  awex::fp8_scale_table_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(amax), static_cast<float*>(scale), n, ue8m0);
  return cudaGetLastError();
}

int awex_launch_fp8_block_dequant(const void* q, const void* scales, void* out, uint64_t rows, uint64_t cols, int64_t q_stride,
                                  int64_t scale_stride, int64_t out_stride, int dst_dtype, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dst_dtype) {
    case 1: return launch_dequant<__nv_bfloat16>(q, scales, out, rows, cols, q_stride, scale_stride, out_stride, s);
    case 2: return launch_dequant<__half>(q, scales, out, rows, cols, q_stride, scale_stride, out_stride, s);
    case 3: return launch_dequant<float>(q, scales, out, rows, cols, q_stride, scale_stride, out_stride, s);
    default: return -3;
  }
}

}  // extern "C"
