// Shared device helpers for the sm_100a kernels of this library.
//
// Every kernel here is launched through an extern "C" function that takes raw
// device pointers, sizes and a CUDA stream; the Python side (csrc/ops.py) checks
// shapes, types and contiguity before it calls.  Element types are passed as an
// integer code so that one entry point serves the bfloat16 and the float32 path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BN_F32 0
#define BN_BF16 1

// Tokens per cache page.  A sequence holds whole pages; position p of a sequence
// lies in page_table[slot][p / BN_PAGE] at row p % BN_PAGE.
#define BN_PAGE 64

// Launch status: 0 ok, otherwise a code that csrc/ops.py turns into an exception.
#define BN_OK 0
#define BN_ERR_BAD_ARG 1
#define BN_ERR_LAUNCH 2

// ---- programmatic dependent launch -----------------------------------------------------------
// Every kernel of this library is launched with programmatic stream serialization: it may start
// while the kernel before it in the stream is still running, and calls pdl_wait() before its
// first access to global memory that another kernel may write (or, for writes, read).  Kernels
// call pdl_launch_dependents() early so that their successor's prologue overlaps them.  What a
// kernel does before pdl_wait() touches only read-only weights, shared and tensor memory.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <utility>
// Compile with -DBN_NO_PDL to serialise kernels completely (for comparisons; csrc/build.py's
// EXTRA_FLAGS); nothing at run time switches it.
#ifdef BN_NO_PDL
static inline bool bn_pdl_enabled() { return false; }
#else
static inline bool bn_pdl_enabled() { return true; }
#endif

// Timestamp probes inside the TMA-fed kernels (where a block's time goes) exist only in builds
// made with -DBN_TRACE; the default build has neither the stores nor the entry points.
#ifdef BN_TRACE
#define BN_TRACE_ONLY(...) __VA_ARGS__
#else
#define BN_TRACE_ONLY(...)
#endif
template <typename... KArgs, typename... Args>
static inline cudaError_t bn_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bn_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
// The same for a grid of thread-block clusters.
template <typename... KArgs, typename... Args>
static inline cudaError_t bn_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bn_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define BN_LAUNCH(kernel, grid, block, smem, stream, ...)                                  \
  do {                                                                                     \
    cudaError_t e__ = bn_launch(kernel, grid, block, smem, stream, __VA_ARGS__);           \
    if (e__ != cudaSuccess) return BN_ERR_LAUNCH + (int)e__;                               \
  } while (0)

#define BN_CHECK_LAUNCH()                                    \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return BN_ERR_LAUNCH + (int)e__; \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// The activation of a gated feed-forward, by code: 0 SiLU, g / (1 + e^-g); 1 the tanh form of GELU,
// 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).  Products with a gated epilogue take the code in
// the bits above the low byte of their `mode` argument (mode 2 | BN_ACT_GELU_TANH << 8).
#define BN_ACT_SILU 0
#define BN_ACT_GELU_TANH 1
__device__ __forceinline__ float glu_activation(float g, int act) {
  if (act == BN_ACT_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.0f + expf(-g));
}

// Load/store of one element of a buffer whose type is only known by code.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == BN_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == BN_F32) ((float*)p)[i] = v;
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dot product of n numbers in shared memory (float32) with a row of weights in global memory, by one
// warp: rows of whole 16-byte pieces are read in such pieces (8 bfloat16 or 4 float32 per lane and
// turn), others number by number.  Every lane gets the result.
__device__ __forceinline__ float warp_dot(const float* __restrict__ xs, const __nv_bfloat16* __restrict__ w, int n, int lane) {
  float acc = 0.f;
  if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int c = lane * 8; c < n; c += 256) {
      uint4 raw = *reinterpret_cast<const uint4*>(w + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h2[i]);
        acc = fmaf(xs[c + 2 * i], f.x, acc);
        acc = fmaf(xs[c + 2 * i + 1], f.y, acc);
      }
    }
  } else {
    for (int c = lane; c < n; c += 32) acc = fmaf(xs[c], __bfloat162float(w[c]), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;
}
__device__ __forceinline__ float warp_dot(const float* __restrict__ xs, const float* __restrict__ w, int n, int lane) {
  float acc = 0.f;
  if ((n & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int c = lane * 4; c < n; c += 128) {
      float4 f = *reinterpret_cast<const float4*>(w + c);
      acc = fmaf(xs[c], f.x, acc);
      acc = fmaf(xs[c + 1], f.y, acc);
      acc = fmaf(xs[c + 2], f.z, acc);
      acc = fmaf(xs[c + 3], f.w, acc);
    }
  } else {
    for (int c = lane; c < n; c += 32) acc = fmaf(xs[c], w[c], acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;
}

// R such dot products at once, of the same numbers with R rows that lie `stride` elements apart: the rows'
// loads are in flight together (a row alone leaves the memory waiting between its few loads).
template <int R>
__device__ __forceinline__ void warp_dot_rows(const float* __restrict__ xs, const __nv_bfloat16* __restrict__ w, size_t stride,
                                              int n, int lane, float* out) {
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  if ((n & 7) == 0 && (stride & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int c = lane * 8; c < n; c += 256) {
      uint4 raw[R];
#pragma unroll
      for (int r = 0; r < R; ++r) raw[r] = *reinterpret_cast<const uint4*>(w + r * stride + c);
      float4 x0 = *reinterpret_cast<const float4*>(xs + c), x1 = *reinterpret_cast<const float4*>(xs + c + 4);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
        float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]), cc = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
        acc[r] = fmaf(x0.x, a.x, acc[r]); acc[r] = fmaf(x0.y, a.y, acc[r]);
        acc[r] = fmaf(x0.z, b.x, acc[r]); acc[r] = fmaf(x0.w, b.y, acc[r]);
        acc[r] = fmaf(x1.x, cc.x, acc[r]); acc[r] = fmaf(x1.y, cc.y, acc[r]);
        acc[r] = fmaf(x1.z, d.x, acc[r]); acc[r] = fmaf(x1.w, d.y, acc[r]);
      }
    }
  } else {
    for (int c = lane; c < n; c += 32)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = fmaf(xs[c], __bfloat162float(w[r * stride + c]), acc[r]);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    out[r] = acc[r];
  }
}
template <int R>
__device__ __forceinline__ void warp_dot_rows(const float* __restrict__ xs, const float* __restrict__ w, size_t stride, int n,
                                              int lane, float* out) {
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  if ((n & 3) == 0 && (stride & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int c = lane * 4; c < n; c += 128) {
      float4 x = *reinterpret_cast<const float4*>(xs + c);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float4 f = *reinterpret_cast<const float4*>(w + r * stride + c);
        acc[r] = fmaf(x.x, f.x, acc[r]); acc[r] = fmaf(x.y, f.y, acc[r]);
        acc[r] = fmaf(x.z, f.z, acc[r]); acc[r] = fmaf(x.w, f.w, acc[r]);
      }
    }
  } else {
    for (int c = lane; c < n; c += 32)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = fmaf(xs[c], w[r * stride + c], acc[r]);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
    out[r] = acc[r];
  }
}

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.
// Every thread gets the result.  The order of additions depends only on the
// block size, never on what else runs, so a row's result does not change with
// the batch around it.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = warp_max(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}

// Address of row (p % BN_PAGE) of key/value head `kvh` in the page that holds position p.
// Cache layout per schedule entry: [n_pages][n_kv_heads][BN_PAGE][head_dim].
__device__ __forceinline__ size_t cache_row_offset(const int* page_table_row, int p,
                                                   int n_kv_heads, int kvh, int head_dim) {
  int page = page_table_row[p / BN_PAGE];
  return (((size_t)page * n_kv_heads + kvh) * BN_PAGE + (p % BN_PAGE)) * (size_t)head_dim;
}
