// SIMT (CUDA-core) kernels of the KAD-Conv path for sm_100a: the general-shape deformable
// convolution (any channel count, fp32/fp16/bf16 storage, fp32 arithmetic) and the pooled 1x1
// projection. Both stage an A tile [32 pixels x K chunk] in shared memory and run the same small
// register-tiled contraction against a weight chunk held in shared memory.
//
// These kernels serve the shapes where tensor cores do not pay (the detector's DSCs have 10-22
// channels) and the float32 configuration, whose 1e-4 max-abs bar rules out TF32.
#include "kad_common.cuh"

namespace kad {
namespace {

constexpr int TP = 32;            // pixels per block (4 warps x 8 pixels)
constexpr int NTHREADS = 128;
constexpr int PPW = 8;            // pixels per warp
constexpr int CC = 16;            // input channels per K chunk of the deformable convolution
constexpr int KC = 9 * CC;        // 144 K values per chunk
constexpr int KPAD = KC + 4;      // row pitch of the A tile (floats), keeps float4 alignment
constexpr int MAXJ = 4;           // output channels per lane -> up to 128 output channels per block

// acc[p][j] += sum_k A[p][k] * Wc[k][lane + 32 j]   for this warp's 8 pixels.
__device__ __forceinline__ void tile_contract(const float* __restrict__ As, const float* __restrict__ Ws,
                                              int kc, int coutT, int J, int lane, int warp,
                                              float (&acc)[PPW][MAXJ]) {
    const float* a0 = As + (warp * PPW) * KPAD;
    for (int k = 0; k < kc; k += 4) {
        float4 s[PPW];
#pragma unroll
        for (int p = 0; p < PPW; ++p) s[p] = *reinterpret_cast<const float4*>(a0 + p * KPAD + k);
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
            if (j < J) {
                int co = lane + 32 * j;
                float w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
                if (co < coutT) {
                    const float* wp = Ws + (size_t)k * coutT + co;
                    w0 = wp[0]; w1 = wp[coutT]; w2 = wp[2 * coutT]; w3 = wp[3 * coutT];
                }
#pragma unroll
                for (int p = 0; p < PPW; ++p) {
                    acc[p][j] = fmaf(s[p].x, w0, acc[p][j]);
                    acc[p][j] = fmaf(s[p].y, w1, acc[p][j]);
                    acc[p][j] = fmaf(s[p].z, w2, acc[p][j]);
                    acc[p][j] = fmaf(s[p].w, w3, acc[p][j]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Deformable 3x3 convolution, NHWC. grid = (ceil(H*W/TP), ceil(Cout/coutT), B).
template <typename T>
__global__ void __launch_bounds__(NTHREADS)
dsc_simt_kernel(const T* __restrict__ x, const void* __restrict__ offset, const void* __restrict__ mask,
                const float* __restrict__ Wt, const float* __restrict__ scale, const float* __restrict__ shift,
                const float* __restrict__ post, void* __restrict__ y, float* __restrict__ gap_partial,
                int H, int W, int Cin, int Cout, int coutT, int offset_f32, int mask_f32, int y_f32, int act) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* As = reinterpret_cast<float*>(smem_raw);                 // [TP][KPAD]
    float* Ws = As + TP * KPAD;                                     // [KC][coutT]
    float* gw = Ws + KC * coutT;                                    // [TP*9][4] corner weights (x mask)
    int* gi = reinterpret_cast<int*>(gw + TP * 9 * 4);              // [TP*9] linear index of corner (y0,x0)
    int* gv = gi + TP * 9;                                          // [TP*9] corner validity bits

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z;
    const int HW = H * W;
    const int p0 = blockIdx.x * TP;
    const int cout0 = blockIdx.y * coutT;
    const int coutHere = min(coutT, Cout - cout0);
    const int J = (coutHere + 31) >> 5;
    const T* xb = x + (size_t)b * HW * Cin;

    // sampling geometry of the block's 32 x 9 samples
    for (int e = tid; e < TP * 9; e += NTHREADS) {
        int p = e / 9, k = e - p * 9;
        int pix = p0 + p;
        float w00 = 0.f, w01 = 0.f, w10 = 0.f, w11 = 0.f;
        int idx = 0, vm = 0;
        if (pix < HW) {
            int py = pix / W, px = pix - py * W;
            size_t ob = ((size_t)b * HW + pix);
            float dy = 0.f, dx = 0.f, m = 1.f;
            if (offset) { dy = load_mixed<T>(offset, ob * 18 + 2 * k, offset_f32); dx = load_mixed<T>(offset, ob * 18 + 2 * k + 1, offset_f32); }
            if (mask) m = load_mixed<T>(mask, ob * 9 + k, mask_f32);
            float sy = (float)(py + k / 3 - 1) + dy;
            float sx = (float)(px + k % 3 - 1) + dx;
            if (sy > -1.f && sy < (float)H && sx > -1.f && sx < (float)W) {
                float fy = floorf(sy), fx = floorf(sx);
                int y0 = (int)fy, x0 = (int)fx;
                float ly = sy - fy, lx = sx - fx, hy = 1.f - ly, hx = 1.f - lx;
                w00 = hy * hx * m; w01 = hy * lx * m; w10 = ly * hx * m; w11 = ly * lx * m;
                idx = y0 * W + x0;
                vm = ((y0 >= 0 && x0 >= 0) ? 1 : 0) | ((y0 >= 0 && x0 + 1 < W) ? 2 : 0) |
                     ((y0 + 1 < H && x0 >= 0) ? 4 : 0) | ((y0 + 1 < H && x0 + 1 < W) ? 8 : 0);
            }
        }
        gw[e * 4 + 0] = w00; gw[e * 4 + 1] = w01; gw[e * 4 + 2] = w10; gw[e * 4 + 3] = w11;
        gi[e] = idx; gv[e] = vm;
    }

    float acc[PPW][MAXJ];
#pragma unroll
    for (int p = 0; p < PPW; ++p)
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) acc[p][j] = 0.f;

    for (int c0 = 0; c0 < Cin; c0 += CC) {
        __syncthreads();   // geometry ready (first pass) / previous chunk consumed
        // weight chunk: Ws[(tap*CC + cl)][co]
        for (int e = tid; e < KC * coutT; e += NTHREADS) {
            int kk = e / coutT, co = e - kk * coutT;
            int tap = kk / CC, cl = kk - tap * CC;
            float v = 0.f;
            if (c0 + cl < Cin && co < coutHere) v = Wt[((size_t)tap * Cin + c0 + cl) * Cout + cout0 + co];
            Ws[e] = v;
        }
        // A tile: bilinear samples x mask
        for (int e = tid; e < TP * 9 * CC; e += NTHREADS) {
            int cl = e % CC, s = e / CC;           // s = pixel*9 + tap
            int p = s / 9, tap = s - p * 9;
            float v = 0.f;
            int vm = gv[s];
            if (vm && c0 + cl < Cin) {
                const T* base = xb + (ptrdiff_t)gi[s] * Cin + c0 + cl;
                const float* w = gw + s * 4;
                if (vm & 1) v = fmaf(w[0], to_f<T>(base[0]), v);
                if (vm & 2) v = fmaf(w[1], to_f<T>(base[Cin]), v);
                if (vm & 4) v = fmaf(w[2], to_f<T>(base[(ptrdiff_t)W * Cin]), v);
                if (vm & 8) v = fmaf(w[3], to_f<T>(base[(ptrdiff_t)(W + 1) * Cin]), v);
            }
            As[p * KPAD + tap * CC + cl] = v;
        }
        __syncthreads();
        tile_contract(As, Ws, KC, coutT, J, lane, warp, acc);
    }

    // epilogue: affine, activation, branch scale; per-block channel sums for the SE squeeze
    float* red = As;   // reuse as [4 warps][coutT]
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
        if (j < J) {
            int co = lane + 32 * j;
            bool live = co < coutHere;
            int cg = cout0 + co;
            float sc = (live && scale) ? scale[cg] : 1.f;
            float sh = (live && shift) ? shift[cg] : 0.f;
            float ps = (live && post) ? post[cg] : 1.f;
            float sum = 0.f;
#pragma unroll
            for (int p = 0; p < PPW; ++p) {
                int pix = p0 + warp * PPW + p;
                if (live && pix < HW) {
                    float v = apply_act(fmaf(acc[p][j], sc, sh), act) * ps;
                    size_t o = ((size_t)b * HW + pix) * Cout + cg;
                    store_mixed<T>(y, o, y_f32, v);
                    // the squeeze must see what the next kernel reads back, i.e. the stored value
                    sum += y_f32 ? v : to_f<T>(from_f<T>(v));
                }
            }
            if (live) red[warp * coutT + co] = sum;
        }
    }
    if (gap_partial) {
        __syncthreads();
        for (int co = tid; co < coutHere; co += NTHREADS) {
            float s = red[co] + red[coutT + co] + red[2 * coutT + co] + red[3 * coutT + co];
            gap_partial[((size_t)b * gridDim.x + blockIdx.x) * Cout + cout0 + co] = s;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// avg-pool (pool x pool, floor) + 1x1 convolution + bias + activation. grid as above over output pixels.
template <typename T>
__global__ void __launch_bounds__(NTHREADS)
pool_project_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                    T* __restrict__ y, int H, int W, int Ho, int Wo, int Cin, int Cout, int coutT,
                    int pool, int act, int x_cs, int y_cs) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* As = reinterpret_cast<float*>(smem_raw);   // [TP][KPAD]
    float* Ws = As + TP * KPAD;                       // [KC][coutT]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.z;
    const int HWo = Ho * Wo;
    const int p0 = blockIdx.x * TP;
    const int cout0 = blockIdx.y * coutT;
    const int coutHere = min(coutT, Cout - cout0);
    const int J = (coutHere + 31) >> 5;
    const float inv = 1.f / (float)(pool * pool);
    const T* xb = x + (size_t)b * H * W * x_cs;

    float acc[PPW][MAXJ];
#pragma unroll
    for (int p = 0; p < PPW; ++p)
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) acc[p][j] = 0.f;

    for (int c0 = 0; c0 < Cin; c0 += KC) {
        int kc = min(KC, Cin - c0);
        int kc4 = (kc + 3) & ~3;
        __syncthreads();
        for (int e = tid; e < kc4 * coutT; e += NTHREADS) {
            int kk = e / coutT, co = e - kk * coutT;
            float v = 0.f;
            if (kk < kc && co < coutHere) v = w[(size_t)(cout0 + co) * Cin + c0 + kk];
            Ws[e] = v;
        }
        for (int e = tid; e < TP * kc4; e += NTHREADS) {
            int kk = e % kc4, p = e / kc4;
            int pix = p0 + p;
            float v = 0.f;
            if (pix < HWo && kk < kc) {
                int yo = pix / Wo, xo = pix - yo * Wo;
                const T* base = xb + ((size_t)(yo * pool) * W + xo * pool) * x_cs + c0 + kk;
                for (int dy = 0; dy < pool; ++dy)
                    for (int dx = 0; dx < pool; ++dx) v += to_f<T>(base[((size_t)dy * W + dx) * x_cs]);
                v *= inv;
            }
            As[p * KPAD + kk] = v;
        }
        __syncthreads();
        tile_contract(As, Ws, kc4, coutT, J, lane, warp, acc);
    }
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
        if (j < J) {
            int co = lane + 32 * j;
            if (co < coutHere) {
                float bb = bias ? bias[cout0 + co] : 0.f;
#pragma unroll
                for (int p = 0; p < PPW; ++p) {
                    int pix = p0 + warp * PPW + p;
                    if (pix < HWo) y[((size_t)b * HWo + pix) * y_cs + cout0 + co] = from_f<T>(apply_act(acc[p][j] + bb, act));
                }
            }
        }
    }
}

template <typename T>
__global__ void pack_dsc_weight_simt_kernel(const float* __restrict__ w, float* __restrict__ dst, int Cin, int Cout) {
    // W[o][i][k] -> dst[k][i][o]
    int n = 9 * Cin * Cout;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n; e += gridDim.x * blockDim.x) {
        int o = e % Cout, r = e / Cout;
        int i = r % Cin, k = r / Cin;
        dst[e] = w[((size_t)o * Cin + i) * 9 + k];
    }
}

inline int pick_cout_tile(int Cout) {
    int t = Cout <= 128 ? Cout : 128;
    return (t + 3) & ~3;
}

}  // namespace

int dsc_px_blocks(int H, int W);
bool dsc_px_supported(int Cin, int Cout);
int launch_dsc_px(const KadDscArgs& a, cudaStream_t st);
bool pool_project_px_supported(int Cin, int Cout);
int launch_pool_project_px(const void* x, const float* w, const float* bias, void* y, int B, int H, int W, int Cin, int Cout,
                           int pool, int act, int x_cs, int y_cs, int dtype, cudaStream_t st);

// number of per-image partial sums the SIMT path writes for the SE squeeze
int dsc_simt_tiles(int H, int W, int Cin, int Cout) {
    return dsc_px_supported(Cin, Cout) ? dsc_px_blocks(H, W) : (H * W + TP - 1) / TP;
}

int launch_dsc_simt(const KadDscArgs& a, cudaStream_t st) {
    if (dsc_px_supported(a.Cin, a.Cout)) return launch_dsc_px(a, st);     // small channel counts: pixel-per-thread kernel
    int coutT = pick_cout_tile(a.Cout);
    size_t smem = sizeof(float) * ((size_t)TP * KPAD + (size_t)KC * coutT + TP * 9 * 4) + sizeof(int) * TP * 9 * 2;
    dim3 grid((a.H * a.W + TP - 1) / TP, (a.Cout + coutT - 1) / coutT, a.B);
    KAD_DISPATCH_DTYPE(a.dtype, {
        auto kern = dsc_simt_kernel<T>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_simt smem attribute: %s", cudaGetErrorString(e));
        kern<<<grid, NTHREADS, smem, st>>>((const T*)a.x, a.offset, a.mask, (const float*)a.weight, a.scale, a.shift,
                                           a.post, a.y, a.gap_partial, a.H, a.W, a.Cin, a.Cout, coutT,
                                           a.offset_f32, a.mask_f32, a.y_f32, a.act);
    });
    KAD_CHECK_LAUNCH("dsc_simt_kernel");
    return KAD_OK;
}

}  // namespace kad

extern "C" int kad_pool_project(const void* x, const float* w, const float* bias, void* y,
                                int B, int H, int W, int Cin, int Cout, int pool, int act,
                                int x_cstride, int y_cstride, int dtype, void* stream) {
    using namespace kad;
    KAD_CHECK_ARG(x && w && y, "kad_pool_project: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && Cin > 0 && Cout > 0, "kad_pool_project: bad shape");
    KAD_CHECK_ARG(pool >= 1 && H / pool > 0 && W / pool > 0, "kad_pool_project: pool %d leaves no output for %dx%d", pool, H, W);
    KAD_CHECK_ARG(x_cstride >= Cin && y_cstride >= Cout, "kad_pool_project: channel stride smaller than channel count");
    if (pool_project_px_supported(Cin, Cout))
        return launch_pool_project_px(x, w, bias, y, B, H, W, Cin, Cout, pool, act, x_cstride, y_cstride, dtype, (cudaStream_t)stream);
    int Ho = H / pool, Wo = W / pool;
    int coutT = pick_cout_tile(Cout);
    size_t smem = sizeof(float) * ((size_t)TP * KPAD + (size_t)KC * coutT);
    dim3 grid((Ho * Wo + TP - 1) / TP, (Cout + coutT - 1) / coutT, B);
    KAD_DISPATCH_DTYPE(dtype, {
        auto kern = pool_project_kernel<T>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "pool_project smem attribute: %s", cudaGetErrorString(e));
        kern<<<grid, NTHREADS, smem, (cudaStream_t)stream>>>((const T*)x, w, bias, (T*)y, H, W, Ho, Wo, Cin, Cout, coutT,
                                                              pool, act, x_cstride, y_cstride);
    });
    KAD_CHECK_LAUNCH("pool_project_kernel");
    return KAD_OK;
}

extern "C" int kad_dsc_pack_weight_simt(const float* w_oihw, float* dst, int Cin, int Cout, void* stream) {
    using namespace kad;
    KAD_CHECK_ARG(w_oihw && dst && Cin > 0 && Cout > 0, "kad_dsc_pack_weight_simt: bad argument");
    int n = 9 * Cin * Cout;
    pack_dsc_weight_simt_kernel<float><<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(w_oihw, dst, Cin, Cout);
    KAD_CHECK_LAUNCH("pack_dsc_weight_simt_kernel");
    return KAD_OK;
}
