// Pixel-per-thread kernels for the small-channel regime of the KAD-Conv path (the detector's DSCs have 10-22
// channels, the offset convolution has 18 outputs): one thread owns one pixel and ALL output channels of its
// group (<= 24, held in registers); the weights sit in shared memory and are read as broadcast float4s, so no
// lane idles on a channel count that is not a multiple of 32 and every weight load feeds four FMAs.
//   dsc_px_kernel           deformable / plain 3x3 convolution + scale/shift/act/post (+ deterministic SE sums)
//   pool_project_px_kernel  avg-pool + 1x1 convolution + bias + activation
// NHWC, fp32 arithmetic, fp32 / fp16 / bf16 storage.
#include "kad_common.cuh"

namespace kad {
namespace {

constexpr int PX_THREADS = 256;
constexpr int PX_MAX_BLOCKS_PER_IMAGE = 64;

// Loads V consecutive channels starting at p (element pointer), as floats.
template <typename T, int V> struct VecLoad;
template <typename T> struct VecLoad<T, 1> {
    static __device__ __forceinline__ void ld(const T* p, float (&o)[1]) { o[0] = to_f<T>(*p); }
};
template <> struct VecLoad<float, 2> {
    static __device__ __forceinline__ void ld(const float* p, float (&o)[2]) { float2 v = *reinterpret_cast<const float2*>(p); o[0] = v.x; o[1] = v.y; }
};
template <> struct VecLoad<float, 4> {
    static __device__ __forceinline__ void ld(const float* p, float (&o)[4]) { float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <> struct VecLoad<__half, 2> {
    static __device__ __forceinline__ void ld(const __half* p, float (&o)[2]) { float2 f = __half22float2(*reinterpret_cast<const __half2*>(p)); o[0] = f.x; o[1] = f.y; }
};
template <> struct VecLoad<__half, 4> {
    static __device__ __forceinline__ void ld(const __half* p, float (&o)[4]) {
        uint2 u = *reinterpret_cast<const uint2*>(p);
        float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
};
template <> struct VecLoad<__nv_bfloat16, 2> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&o)[2]) { float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); o[0] = f.x; o[1] = f.y; }
};
template <> struct VecLoad<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&o)[4]) {
        uint2 u = *reinterpret_cast<const uint2*>(p);
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
    }
};

// acc[0..4*NCO4) += s * W[row][0..4*NCO4), the weight row read as broadcast float4s
template <int NCO4>
__device__ __forceinline__ void fma_row(float (&acc)[4 * NCO4], float s, const float4* __restrict__ wrow) {
#pragma unroll
    for (int q = 0; q < NCO4; ++q) {
        const float4 w = wrow[q];
        acc[4 * q + 0] = fmaf(s, w.x, acc[4 * q + 0]); acc[4 * q + 1] = fmaf(s, w.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(s, w.z, acc[4 * q + 2]); acc[4 * q + 3] = fmaf(s, w.w, acc[4 * q + 3]);
    }
}

// One tap of one pixel: bilinear sample of V channels at a time, folded into the accumulators.
template <typename T, int NCO4, int V>
__device__ __forceinline__ void tap_accumulate(float (&acc)[4 * NCO4], const T* __restrict__ base, int Cin, int W, int vm,
                                               float w00, float w01, float w10, float w11, const float4* __restrict__ wtap) {
    const ptrdiff_t dx = Cin, dy = (ptrdiff_t)W * Cin;
    for (int c0 = 0; c0 < Cin; c0 += V) {
        float s[V];
#pragma unroll
        for (int v = 0; v < V; ++v) s[v] = 0.f;
        float t[V];
        if (vm & 1) { VecLoad<T, V>::ld(base + c0, t);
#pragma unroll
            for (int v = 0; v < V; ++v) s[v] = fmaf(w00, t[v], s[v]); }
        if (vm & 2) { VecLoad<T, V>::ld(base + dx + c0, t);
#pragma unroll
            for (int v = 0; v < V; ++v) s[v] = fmaf(w01, t[v], s[v]); }
        if (vm & 4) { VecLoad<T, V>::ld(base + dy + c0, t);
#pragma unroll
            for (int v = 0; v < V; ++v) s[v] = fmaf(w10, t[v], s[v]); }
        if (vm & 8) { VecLoad<T, V>::ld(base + dy + dx + c0, t);
#pragma unroll
            for (int v = 0; v < V; ++v) s[v] = fmaf(w11, t[v], s[v]); }
#pragma unroll
        for (int v = 0; v < V; ++v) fma_row<NCO4>(acc, s[v], wtap + (size_t)(c0 + v) * NCO4);
    }
}

// grid = (blocks per image, output-channel groups, B). Each block owns the pixels p = blockIdx.x*256 + tid + k*gridDim.x*256.
template <typename T, int NCO4>
__global__ void __launch_bounds__(PX_THREADS)
dsc_px_kernel(const T* __restrict__ x, const void* __restrict__ offset, const void* __restrict__ mask,
              const float* __restrict__ Wt, const float* __restrict__ scale, const float* __restrict__ shift,
              const float* __restrict__ post, void* __restrict__ y, float* __restrict__ gap_partial,
              int H, int W, int Cin, int Cout, int vec, int offset_f32, int mask_f32, int y_f32, int act) {
    constexpr int COP = 4 * NCO4;
    extern __shared__ __align__(16) float smem_px[];
    float* Ws = smem_px;                       // [9][Cin][COP]
    float* ep = Ws + 9 * Cin * COP;            // scale | shift | post, [COP] each
    float* red = ep + 3 * COP;                 // [8 warps][COP]
    const int tid = threadIdx.x, b = blockIdx.z, HW = H * W;
    const int cout0 = blockIdx.y * COP, coutHere = min(COP, Cout - cout0);
    for (int e = tid; e < 9 * Cin * COP; e += PX_THREADS) {
        const int co = e % COP, r = e / COP;   // r = tap*Cin + ci
        Ws[e] = co < coutHere ? Wt[(size_t)r * Cout + cout0 + co] : 0.f;
    }
    for (int e = tid; e < COP; e += PX_THREADS) {
        const bool live = e < coutHere;
        ep[e] = (live && scale) ? scale[cout0 + e] : 1.f;
        ep[COP + e] = (live && shift) ? shift[cout0 + e] : 0.f;
        ep[2 * COP + e] = (live && post) ? post[cout0 + e] : 1.f;
    }
    __syncthreads();
    const float4* Ws4 = reinterpret_cast<const float4*>(Ws);
    const T* xb = x + (size_t)b * HW * Cin;
    float psum[COP];
#pragma unroll
    for (int i = 0; i < COP; ++i) psum[i] = 0.f;

    for (int pix = blockIdx.x * PX_THREADS + tid; pix < HW; pix += gridDim.x * PX_THREADS) {
        const int py = pix / W, px = pix - py * W;
        const size_t gp = (size_t)b * HW + pix;
        float acc[COP];
#pragma unroll
        for (int i = 0; i < COP; ++i) acc[i] = 0.f;
#pragma unroll 1
        for (int k = 0; k < 9; ++k) {
            float dy = 0.f, dx = 0.f, m = 1.f;
            if (offset) { dy = load_mixed<T>(offset, gp * 18 + 2 * k, offset_f32); dx = load_mixed<T>(offset, gp * 18 + 2 * k + 1, offset_f32); }
            if (mask) m = load_mixed<T>(mask, gp * 9 + k, mask_f32);
            const float sy = (float)(py + k / 3 - 1) + dy, sx = (float)(px + k % 3 - 1) + dx;
            if (!(sy > -1.f && sy < (float)H && sx > -1.f && sx < (float)W)) continue;
            const float fy = floorf(sy), fx = floorf(sx);
            const int y0 = (int)fy, x0 = (int)fx;
            const float ly = sy - fy, lx = sx - fx, hy = 1.f - ly, hx = 1.f - lx;
            int vm = ((y0 >= 0 && x0 >= 0) ? 1 : 0) | ((y0 >= 0 && x0 + 1 < W) ? 2 : 0) |
                     ((y0 + 1 < H && x0 >= 0) ? 4 : 0) | ((y0 + 1 < H && x0 + 1 < W) ? 8 : 0);
            const float w00 = hy * hx * m, w01 = hy * lx * m, w10 = ly * hx * m, w11 = ly * lx * m;
            if (!offset) vm &= 1;              // integer sample position: only the first corner has weight
            if (!vm) continue;
            const T* base = xb + ((ptrdiff_t)y0 * W + x0) * Cin;
            const float4* wtap = Ws4 + (size_t)k * Cin * NCO4;
            if (vec == 4) tap_accumulate<T, NCO4, 4>(acc, base, Cin, W, vm, w00, w01, w10, w11, wtap);
            else if (vec == 2) tap_accumulate<T, NCO4, 2>(acc, base, Cin, W, vm, w00, w01, w10, w11, wtap);
            else tap_accumulate<T, NCO4, 1>(acc, base, Cin, W, vm, w00, w01, w10, w11, wtap);
        }
        const size_t ob = gp * Cout + cout0;
#pragma unroll
        for (int i = 0; i < COP; ++i) {
            if (i < coutHere) {
                const float v = apply_act(fmaf(acc[i], ep[i], ep[COP + i]), act) * ep[2 * COP + i];
                store_mixed<T>(y, ob + i, y_f32, v);
                psum[i] += y_f32 ? v : to_f<T>(from_f<T>(v));      // sums of what the next kernel reads back
            }
        }
    }
    if (gap_partial) {
        const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
        for (int i = 0; i < COP; ++i) {
            float v = psum[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp * COP + i] = v;
        }
        __syncthreads();
        if (tid < coutHere) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < PX_THREADS / 32; ++w) s += red[w * COP + tid];
            gap_partial[((size_t)b * gridDim.x + blockIdx.x) * Cout + cout0 + tid] = s;
        }
    }
}

// avg-pool (pool x pool, floor) + 1x1 conv + bias + act; same thread <-> pixel mapping.
template <typename T, int NCO4, int V>
__device__ __forceinline__ void pool_accumulate(float (&acc)[4 * NCO4], const T* __restrict__ base, int Cin, int W, int x_cs, int pool,
                                                float inv, const float4* __restrict__ Ws4) {
    for (int c0 = 0; c0 < Cin; c0 += V) {
        float s[V];
#pragma unroll
        for (int v = 0; v < V; ++v) s[v] = 0.f;
        for (int dy = 0; dy < pool; ++dy)
            for (int dx = 0; dx < pool; ++dx) {
                float t[V];
                VecLoad<T, V>::ld(base + ((size_t)dy * W + dx) * x_cs + c0, t);
#pragma unroll
                for (int v = 0; v < V; ++v) s[v] += t[v];
            }
#pragma unroll
        for (int v = 0; v < V; ++v) fma_row<NCO4>(acc, s[v] * inv, Ws4 + (size_t)(c0 + v) * NCO4);
    }
}

template <typename T, int NCO4>
__global__ void __launch_bounds__(PX_THREADS)
pool_project_px_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, T* __restrict__ y,
                       int H, int W, int Ho, int Wo, int Cin, int Cout, int pool, int act, int x_cs, int y_cs, int vec) {
    constexpr int COP = 4 * NCO4;
    extern __shared__ __align__(16) float smem_px[];
    float* Ws = smem_px;                       // [Cin][COP]
    float* bs = Ws + Cin * COP;                // [COP]
    const int tid = threadIdx.x, b = blockIdx.z, HWo = Ho * Wo;
    const int cout0 = blockIdx.y * COP, coutHere = min(COP, Cout - cout0);
    for (int e = tid; e < Cin * COP; e += PX_THREADS) {
        const int co = e % COP, ci = e / COP;
        Ws[e] = co < coutHere ? w[(size_t)(cout0 + co) * Cin + ci] : 0.f;
    }
    for (int e = tid; e < COP; e += PX_THREADS) bs[e] = (e < coutHere && bias) ? bias[cout0 + e] : 0.f;
    __syncthreads();
    const float4* Ws4 = reinterpret_cast<const float4*>(Ws);
    const float inv = 1.f / (float)(pool * pool);
    const T* xb = x + (size_t)b * H * W * x_cs;
    for (int pix = blockIdx.x * PX_THREADS + tid; pix < HWo; pix += gridDim.x * PX_THREADS) {
        const int yo = pix / Wo, xo = pix - yo * Wo;
        const T* base = xb + ((size_t)(yo * pool) * W + xo * pool) * x_cs;
        float acc[COP];
#pragma unroll
        for (int i = 0; i < COP; ++i) acc[i] = bs[i];
        if (vec == 4) pool_accumulate<T, NCO4, 4>(acc, base, Cin, W, x_cs, pool, inv, Ws4);
        else if (vec == 2) pool_accumulate<T, NCO4, 2>(acc, base, Cin, W, x_cs, pool, inv, Ws4);
        else pool_accumulate<T, NCO4, 1>(acc, base, Cin, W, x_cs, pool, inv, Ws4);
        T* dst = y + ((size_t)b * HWo + pix) * y_cs + cout0;
#pragma unroll
        for (int i = 0; i < COP; ++i)
            if (i < coutHere) dst[i] = from_f<T>(apply_act(acc[i], act));
    }
}

// vector width (elements) usable for channel loads: the channel count / strides and the base must keep the alignment
inline int pick_vec(int c_elems, int stride_elems, const void* base, size_t elem) {
    for (int v = 4; v >= 2; v >>= 1)
        if (c_elems % v == 0 && stride_elems % v == 0 && ((uintptr_t)base % (v * elem)) == 0) return v;
    return 1;
}

inline int pick_nco4(int Cout) {
    // groups of at most 24 output channels; pick the group size that wastes the least
    int groups = (Cout + 23) / 24;
    int per = (Cout + groups - 1) / groups;
    int n = (per + 3) / 4;
    return n < 3 ? 3 : n;     // 12, 16, 20 or 24 channels per group
}

}  // namespace

int dsc_px_blocks(int H, int W) {
    int n = (H * W + PX_THREADS - 1) / PX_THREADS;
    return n < 1 ? 1 : (n > PX_MAX_BLOCKS_PER_IMAGE ? PX_MAX_BLOCKS_PER_IMAGE : n);
}

bool dsc_px_supported(int Cin, int Cout) { return Cin <= 64; }

int launch_dsc_px(const KadDscArgs& a, cudaStream_t st) {
    const int nco4 = pick_nco4(a.Cout), COP = 4 * nco4;
    const int groups = (a.Cout + COP - 1) / COP;
    size_t smem = sizeof(float) * ((size_t)9 * a.Cin * COP + 3 * COP + 8 * COP);
    dim3 grid(dsc_px_blocks(a.H, a.W), groups, a.B);
    const int vec = pick_vec(a.Cin, a.Cin, a.x, dtype_size(a.dtype));
#define KAD_PX_LAUNCH(N)                                                                                              \
    {                                                                                                                 \
        auto kern = dsc_px_kernel<T, N>;                                                                              \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_px smem attribute: %s", cudaGetErrorString(e));          \
        kern<<<grid, PX_THREADS, smem, st>>>((const T*)a.x, a.offset, a.mask, (const float*)a.weight, a.scale, a.shift, a.post, a.y, \
                                             a.gap_partial, a.H, a.W, a.Cin, a.Cout, vec, a.offset_f32, a.mask_f32, a.y_f32, a.act); \
    }
    KAD_DISPATCH_DTYPE(a.dtype, {
        switch (nco4) {
            case 3: KAD_PX_LAUNCH(3) break;
            case 4: KAD_PX_LAUNCH(4) break;
            case 5: KAD_PX_LAUNCH(5) break;
            default: KAD_PX_LAUNCH(6) break;
        }
    });
#undef KAD_PX_LAUNCH
    KAD_CHECK_LAUNCH("dsc_px_kernel");
    return KAD_OK;
}

bool pool_project_px_supported(int Cin, int Cout) { return Cin <= 512 && Cout <= 96; }

int launch_pool_project_px(const void* x, const float* w, const float* bias, void* y, int B, int H, int W, int Cin, int Cout,
                           int pool, int act, int x_cs, int y_cs, int dtype, cudaStream_t st) {
    const int nco4 = pick_nco4(Cout), COP = 4 * nco4;
    const int groups = (Cout + COP - 1) / COP;
    const int Ho = H / pool, Wo = W / pool;
    size_t smem = sizeof(float) * ((size_t)Cin * COP + COP);
    int bx = (Ho * Wo + PX_THREADS - 1) / PX_THREADS;
    if (bx > 4 * PX_MAX_BLOCKS_PER_IMAGE) bx = 4 * PX_MAX_BLOCKS_PER_IMAGE;
    dim3 grid(bx, groups, B);
    const int vec = pick_vec(Cin, x_cs, x, dtype_size(dtype));
#define KAD_PP_LAUNCH(N)                                                                                              \
    {                                                                                                                 \
        auto kern = pool_project_px_kernel<T, N>;                                                                     \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "pool_project_px smem attribute: %s", cudaGetErrorString(e)); \
        kern<<<grid, PX_THREADS, smem, st>>>((const T*)x, w, bias, (T*)y, H, W, Ho, Wo, Cin, Cout, pool, act, x_cs, y_cs, vec); \
    }
    KAD_DISPATCH_DTYPE(dtype, {
        switch (nco4) {
            case 3: KAD_PP_LAUNCH(3) break;
            case 4: KAD_PP_LAUNCH(4) break;
            case 5: KAD_PP_LAUNCH(5) break;
            default: KAD_PP_LAUNCH(6) break;
        }
    });
#undef KAD_PP_LAUNCH
    KAD_CHECK_LAUNCH("pool_project_px_kernel");
    return KAD_OK;
}

}  // namespace kad
