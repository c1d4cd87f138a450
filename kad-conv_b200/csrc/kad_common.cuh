// Shared helpers for the kadconv_b200 kernels: storage-type load/store, error reporting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "../../include/kadconv_b200.h"

namespace kad {

// ---- error reporting (thread-local, never throws) ------------------------------------------------
std::string& last_error();
int fail(int code, const char* fmt, ...);

#define KAD_CHECK_ARG(cond, ...) do { if (!(cond)) return kad::fail(KAD_ERR_INVALID, __VA_ARGS__); } while (0)
#define KAD_CHECK_LAUNCH(what) do { cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) return kad::fail(KAD_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e_)); } while (0)

// ---- programmatic dependent launch ----------------------------------------------------------------------
// launch_pdl: the grid may be scheduled while the kernel before it in the stream is still draining (once every block of that
// kernel has called grid_dependents_go() or has ended), so its launch latency and whatever it does before grid_dependency_wait()
// (staging weights, setting up barriers) overlap that kernel's tail. A kernel launched this way MUST call grid_dependency_wait()
// before it reads or writes anything another kernel touches: the wait returns when the kernels before it have completed and
// their writes are visible. Both instructions do nothing in a kernel launched the ordinary way, and the pair is recorded as a
// programmatic edge when the launch is captured into a CUDA graph.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_go() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- storage types -----------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Reads element i of a buffer that is float32 when `f32` is set and T otherwise.
template <typename T>
__device__ __forceinline__ float load_mixed(const void* p, size_t i, int f32) {
    return f32 ? reinterpret_cast<const float*>(p)[i] : to_f<T>(reinterpret_cast<const T*>(p)[i]);
}
template <typename T>
__device__ __forceinline__ void store_mixed(void* p, size_t i, int f32, float v) {
    if (f32) reinterpret_cast<float*>(p)[i] = v; else reinterpret_cast<T*>(p)[i] = from_f<T>(v);
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }
// The LCSA modulation mask (nine per pixel): hardware exponential and reciprocal, about 2 ulp of float32 on a value in (0, 1), i.e.
// below 1e-6 absolute. Every kernel that produces a mask uses this one, so the forms stay bit-identical among themselves.
__device__ __forceinline__ float sigmoid_mask(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }
// SiLU for the 16-bit epilogues: v / (1 + 2^(-v * log2 e)) with the hardware exponential and reciprocal (two
// special-function instructions, about 2 ulp of float32: far below the rounding of the 16-bit store that follows).
// Building with -DKAD_SILU_TANH selects v * (0.5 * tanh.approx(v / 2) + 0.5) instead: one special-function
// instruction, but about 5e-4 relative error, the size of a half-precision rounding step, on every activation.
__device__ __forceinline__ float silu_fast(float v) {
#ifdef KAD_SILU_TANH
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * v));
    return v * fmaf(0.5f, th, 0.5f);
#else
    return __fdividef(v, 1.0f + __expf(-v));
#endif
}
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == KAD_ACT_SILU) return v * sigmoidf_(v);
    if (act == KAD_ACT_RELU) return fmaxf(v, 0.0f);
    return v;
}

inline size_t dtype_size(int dtype) { return dtype == KAD_F32 ? 4 : 2; }

// kad_elementwise.cu: second stage of the LCSA from prepared operands (used by the layer call when the pyramid kernel has
// finished the first stage in its tail)
int lcsa_mask_from_prepared(const float* rows, int rows_are_means, const float* A, const float* Sm,
                            const float* w2, const float* b2, const float* w3, const float* b3,
                            void* mask, int B, int H, int W, int C, int mask_f32, int dtype, cudaStream_t st);

// Dispatch a templated launcher on the storage type.
#define KAD_DISPATCH_DTYPE(dtype, ...)                                                   \
    switch (dtype) {                                                                     \
        case KAD_F32:  { using T = float;          __VA_ARGS__; break; }                 \
        case KAD_F16:  { using T = __half;         __VA_ARGS__; break; }                 \
        case KAD_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; }                 \
        default: return kad::fail(KAD_ERR_INVALID, "unknown dtype %d", (int)(dtype));    \
    }

}  // namespace kad
