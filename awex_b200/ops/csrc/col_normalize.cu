// Column-wise L2 normalisation of a row-major 2-D tensor for sm_100a:
//     out[r, c] = x[r, c] / max(||x[:, c]||_2, eps)
// which is torch.nn.functional.normalize(x, dim=0, p=2, eps) (the published
// language-model head of architectures that set `norm_head`; reference:
// awex/converter/mcore_converter.py:668-675, one ATen norm + clamp + expand +
// divide with two temporaries of the tensor's size per update).
//
// Three launches, no atomics, so the result does not depend on scheduling:
//   1. partial sums of squares per (band of rows, column) in fp32, 8 columns per
//      thread from one 16-byte load per row, rows of a band added in order;
//   2. per column, the bands' partial sums added in band order, the norm rounded
//      to the tensor's dtype (as the ATen op returns it) and clamped to eps;
//   3. every element divided by its column's norm (a true division, rounded to
//      the tensor's dtype), 16-byte loads and stores.
// The sums are accumulated in another order than ATen's, so a norm can differ
// from it in the last bit of the tensor's dtype; everything else is identical.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

namespace awex {

constexpr int kNormThreads = 128;
constexpr int kBandRows = 256;

template <typename T>
struct Pack {  // 16 bytes of T
  static constexpr int kN = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, float* v) {
  if constexpr (std::is_same<T, float>::value) {
    v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y); v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
  } else {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ float round_to(float x) {
  if constexpr (std::is_same<T, float>::value) return x;
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) return __bfloat162float(__float2bfloat16_rn(x));
  else return __half2float(__float2half_rn(x));
}

// grid: (column groups, bands); partial[band, col]
template <typename T>
__global__ void __launch_bounds__(kNormThreads) col_sumsq_kernel(const T* __restrict__ x, float* __restrict__ partial, uint32_t rows,
                                                                uint32_t cols, int64_t stride) {
  constexpr int kN = Pack<T>::kN;
  const uint32_t c0 = (blockIdx.x * kNormThreads + threadIdx.x) * kN;
  if (c0 >= cols) return;
  const uint32_t r0 = blockIdx.y * kBandRows, r1 = min(r0 + kBandRows, rows);
  float acc[kN];
#pragma unroll
  for (int i = 0; i < kN; ++i) acc[i] = 0.f;
  const bool whole = c0 + kN <= cols;
  for (uint32_t r = r0; r < r1; ++r) {
    const T* row = x + static_cast<int64_t>(r) * stride + c0;
    float v[kN];
    if (whole && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      unpack16<T>(__ldg(reinterpret_cast<const uint4*>(row)), v);
    } else {
#pragma unroll
      for (int i = 0; i < kN; ++i) v[i] = (c0 + i < cols) ? static_cast<float>(row[i]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < kN; ++i) acc[i] = fmaf(v[i], v[i], acc[i]);
  }
  float* out = partial + static_cast<int64_t>(blockIdx.y) * cols + c0;
#pragma unroll
  for (int i = 0; i < kN; ++i)
    if (c0 + i < cols) out[i] = acc[i];
}

template <typename T>
__global__ void col_norm_finish_kernel(const float* __restrict__ partial, float* __restrict__ norms, uint32_t bands, uint32_t cols, float eps) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (uint32_t b = 0; b < bands; ++b) s += partial[static_cast<int64_t>(b) * cols + c];
  const float n = round_to<T>(sqrtf(s));
  norms[c] = n < eps ? eps : n;  // NaN stays NaN
}

template <typename T>
__global__ void __launch_bounds__(256) col_scale_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ norms,
                                                        uint32_t rows, uint32_t cols, int64_t x_stride, int64_t out_stride) {
  constexpr int kN = Pack<T>::kN;
  const uint32_t groups = (cols + kN - 1) / kN;
  const uint64_t total = static_cast<uint64_t>(rows) * groups;
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint32_t r = static_cast<uint32_t>(i / groups), c0 = static_cast<uint32_t>(i % groups) * kN;
    const T* src = x + static_cast<int64_t>(r) * x_stride + c0;
    T* dst = out + static_cast<int64_t>(r) * out_stride + c0;
    const bool whole = c0 + kN <= cols;
    float v[kN];
    if (whole && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      unpack16<T>(__ldg(reinterpret_cast<const uint4*>(src)), v);
    } else {
#pragma unroll
      for (int j = 0; j < kN; ++j) v[j] = (c0 + j < cols) ? static_cast<float>(src[j]) : 0.f;
    }
    T q[kN];
#pragma unroll
    for (int j = 0; j < kN; ++j) {
      const float d = (c0 + j < cols) ? norms[c0 + j] : 1.f;
      const float f = __fdiv_rn(v[j], d);
      if constexpr (std::is_same<T, float>::value) q[j] = f;
      else if constexpr (std::is_same<T, __nv_bfloat16>::value) q[j] = __float2bfloat16_rn(f);
      else q[j] = __float2half_rn(f);
    }
    if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(q);
    } else {
      for (int j = 0; j < kN; ++j)
        if (c0 + j < cols) dst[j] = q[j];
    }
  }
}

template <typename T>
int launch_col_normalize(const void* x, void* out, void* scratch, uint32_t rows, uint32_t cols, int64_t x_stride, int64_t out_stride,
                         float eps, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  constexpr int kN = Pack<T>::kN;
  const uint32_t bands = (rows + kBandRows - 1) / kBandRows;
  float* partial = static_cast<float*>(scratch);
  float* norms = partial + static_cast<int64_t>(bands) * cols;
  const dim3 grid1((cols + kNormThreads * kN - 1) / (kNormThreads * kN), bands);
  col_sumsq_kernel<T><<<grid1, kNormThreads, 0, s>>>(static_cast<const T*>(x), partial, rows, cols, x_stride);
  col_norm_finish_kernel<T><<<(cols + 255) / 256, 256, 0, s>>>(partial, norms, bands, cols, eps);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const uint64_t work = static_cast<uint64_t>(rows) * ((cols + kN - 1) / kN);
  uint64_t grid3 = (work + 255) / 256;
  if (grid3 > static_cast<uint64_t>(sms) * 16) grid3 = static_cast<uint64_t>(sms) * 16;
  col_scale_kernel<T><<<static_cast<unsigned>(grid3), 256, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out), norms, rows, cols,
                                                                   x_stride, out_stride);
  return cudaGetLastError();
}

}  // namespace awex

extern "C" {

// Floats of scratch the launcher needs for a [rows, cols] tensor.
uint64_t awex_col_normalize_scratch_floats(uint64_t rows, uint64_t cols) {
  return ((rows + awex::kBandRows - 1) / awex::kBandRows + 1) * cols;
}

// dtype codes: 1 bf16, 2 f16, 3 f32.  Strides in elements.  `out` may be `x`.
int awex_launch_col_l2_normalize(const void* x, void* out, void* scratch, uint64_t rows, uint64_t cols, int64_t x_stride,
                                 int64_t out_stride, int dtype, float eps, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows > 0xFFFFFFFFull || cols > 0xFFFFFFFFull) return cudaErrorInvalidValue;
  switch (dtype) {
    case 1: return awex::launch_col_normalize<__nv_bfloat16>(x, out, scratch, rows, cols, x_stride, out_stride, eps, s);
    case 2: return awex::launch_col_normalize<__half>(x, out, scratch, rows, cols, x_stride, out_stride, eps, s);
    case 3: return awex::launch_col_normalize<float>(x, out, scratch, rows, cols, x_stride, out_stride, eps, s);
    default: return -3;
  }
}

}  // extern "C"
