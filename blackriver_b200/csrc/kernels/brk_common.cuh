// Shared device helpers for the sm_100a kernel library: 128-bit vector access for fp32/fp16
// storage, warp/block reductions, launch-error capture.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "brk.h"

namespace brk {

void set_cuda_error(cudaError_t e, const char* where);
// Records a plain message for brk_last_cuda_error() (argument errors that deserve an explanation).
void set_error_message(const std::string& msg);

// Checks the launch that just happened; records the message for brk_last_cuda_error().
inline int launch_status(const char* where) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e, where);
        return BRK_CUDA_ERROR;
    }
    return BRK_OK;
}

int sm_count();

// ---------------------------------------------------------------------------------------
// 16-byte packets.  Vec<T>::N elements of T per packet; load/store go through one
// ld.global.v4 / st.global.v4.
// ---------------------------------------------------------------------------------------
template <typename T>
struct Vec;

template <>
struct Vec<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void unpack(const uint4& t) {
        v[0] = __uint_as_float(t.x); v[1] = __uint_as_float(t.y); v[2] = __uint_as_float(t.z); v[3] = __uint_as_float(t.w);
    }
    __device__ __forceinline__ uint4 pack() const {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
    __device__ __forceinline__ void load(const float* p) {
        float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void load_stream(const float* p) {
        float4 t = __ldcs(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    __device__ __forceinline__ void store_stream(float* p) const {
        __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    }
};

template <>
struct Vec<__half> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void unpack(const uint4& t) {
        const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    __device__ __forceinline__ uint4 pack() const {
        uint4 t;
        __half2* h = reinterpret_cast<__half2*>(&t);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        return t;
    }
    __device__ __forceinline__ void load(const __half* p) { unpack(*reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void load_stream(const __half* p) { unpack(__ldcs(reinterpret_cast<const uint4*>(p))); }
    __device__ __forceinline__ void store(__half* p) const { *reinterpret_cast<uint4*>(p) = pack(); }
    __device__ __forceinline__ void store_stream(__half* p) const { __stcs(reinterpret_cast<uint4*>(p), pack()); }
};

// Raw 16-byte packet loads (kept packed in registers until Vec<T>::unpack).
template <typename T>
__device__ __forceinline__ uint4 ld_raw(const T* p) { return *reinterpret_cast<const uint4*>(p); }
template <typename T>
__device__ __forceinline__ uint4 ld_raw_stream(const T* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

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

// Block-wide sum of up to 2 values at once; `red` is >= 2*32 floats of shared memory.  All
// threads of the block must call it; every thread receives the totals.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    a = warp_sum(a);
    b = warp_sum(b);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();  // protect `red` from the previous use
    if (lane == 0) {
        red[warp] = a;
        red[32 + warp] = b;
    }
    __syncthreads();
    float ta = lane < nwarp ? red[lane] : 0.0f;
    float tb = lane < nwarp ? red[32 + lane] : 0.0f;
    a = warp_sum(ta);
    b = warp_sum(tb);
}

__device__ __forceinline__ float block_max(float a, float* red) {
    a = warp_max(a);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = a;
    __syncthreads();
    float t = lane < nwarp ? red[lane] : -INFINITY;
    return warp_max(t);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch as a programmatic dependent of the kernel before it in the stream: the launch itself overlaps that kernel's
// tail.  Every kernel launched this way executes pdl_wait() before it touches global memory.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace brk
