// Bandwidth-bound kernels of the KAD-Conv path: layout conversion, the LCSA mask branch, the SE
// squeeze / excite / rescale, and the upsample + concat + residual tail. All NHWC, fp32 arithmetic.
#include <mutex>

#include "kad_common.cuh"

namespace kad {
namespace {

// ------------------------------------------------------------------------------ layout conversion
// Per image: src is a [R][S] matrix, dst the [S][R] transpose. NCHW->NHWC: R = C, S = H*W.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int R, int S) {
    __shared__ T tile[32][33];
    const T* s = src + (size_t)blockIdx.z * R * S;
    T* d = dst + (size_t)blockIdx.z * R * S;
    int s0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int r = r0 + i, c = s0 + threadIdx.x;
        if (r < R && c < S) tile[i][threadIdx.x] = s[(size_t)r * S + c];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int c = s0 + i, r = r0 + threadIdx.x;
        if (r < R && c < S) d[(size_t)c * R + r] = tile[threadIdx.x][i];
    }
}

// ------------------------------------------------------------------------------ LCSA
// Row sums over x: grid (H, B), 256 threads.
template <typename T>
__global__ void lcsa_rowsum_kernel(const T* __restrict__ x, float* __restrict__ rowsum, int H, int W, int C) {
    __shared__ float red[256];
    int b = blockIdx.y, h = blockIdx.x, t = threadIdx.x;
    int nC = min(C, 256), lpc = 256 / nC;
    const T* row = x + ((size_t)b * H + h) * W * C;
    for (int cb = 0; cb < C; cb += nC) {
        int cl = t % nC, wl = t / nC, c = cb + cl;
        float acc = 0.f;
        if (wl < lpc && c < C)
            for (int w = wl; w < W; w += lpc) acc += to_f<T>(row[(size_t)w * C + c]);
        red[t] = acc;
        __syncthreads();
        if (t < nC && c < C) {
            float s = 0.f;
            for (int l = 0; l < lpc; ++l) s += red[l * nC + t];
            rowsum[((size_t)b * H + h) * C + c] = s;
        }
        __syncthreads();
    }
}

// Column sums over y: one thread per (x, c), consecutive threads read consecutive addresses.
template <typename T>
__global__ void lcsa_colsum_kernel(const T* __restrict__ x, float* __restrict__ colsum, int H, int W, int C) {
    int b = blockIdx.y;
    int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= W * C) return;
    const T* p = x + (size_t)b * H * W * C + e;
    float acc = 0.f;
    for (int h = 0; h < H; ++h) acc += to_f<T>(p[(size_t)h * W * C]);
    colsum[(size_t)b * W * C + e] = acc;
}

// The 1x11 convolution of (rowmean[h] + colmean[w]) separates (zero padding makes the tap sum depend
// on w): conv = rowmean[h] * S[w] + Cc[w]. With the folded BatchNorm (m, a):
//   h1[b,h,w,c] = relu(rowmean[b,h,c] * Sm[c,w] + A[b,c,w]),  Sm = S*m,  A = (Cc + b1)*m + a.
__global__ void lcsa_prep_kernel(const float* __restrict__ colsum, const float* __restrict__ w1,
                                 const float* __restrict__ b1, const float* __restrict__ bn_m,
                                 const float* __restrict__ bn_a, float* __restrict__ A, float* __restrict__ Sm,
                                 int H, int W, int C) {
    int b = blockIdx.y;
    int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= W * C) return;
    int c = e / W, w = e - c * W;
    float invH = 1.f / (float)H;
    float conv = 0.f, S = 0.f;
#pragma unroll
    for (int k = 0; k < 11; ++k) {
        int ww = w + k - 5;
        if (ww >= 0 && ww < W) {
            float wk = w1[c * 11 + k];
            conv = fmaf(wk, colsum[((size_t)b * W + ww) * C + c] * invH, conv);
            S += wk;
        }
    }
    float m = bn_m[c];
    A[((size_t)b * C + c) * W + w] = (conv + b1[c]) * m + bn_a[c];
    if (b == 0) Sm[(size_t)c * W + w] = S * m;
}

// grid (ceil(W/128), H, B), 128 threads; each thread one pixel.
template <typename T>
__global__ void __launch_bounds__(128)
lcsa_mask_kernel(const float* __restrict__ rowsum, const float* __restrict__ A, const float* __restrict__ Sm,
                 const float* __restrict__ w2, const float* __restrict__ b2, const float* __restrict__ w3,
                 const float* __restrict__ b3, void* __restrict__ mask, int H, int W, int C, int mask_f32) {
    extern __shared__ float sm[];
    float* rm = sm;               // [11][C] row means of rows h-5..h+5 (0 outside the image)
    float* sw2 = rm + 11 * C;     // [C][11]
    float* sw3 = sw2 + 11 * C;    // [9][C]
    float* sb2 = sw3 + 9 * C;     // [C]
    int b = blockIdx.z, h = blockIdx.y, t = threadIdx.x;
    float invW = 1.f / (float)W;
    for (int e = t; e < 11 * C; e += 128) {
        int k = e / C, c = e - k * C, hh = h + k - 5;
        rm[e] = (hh >= 0 && hh < H) ? rowsum[((size_t)b * H + hh) * C + c] * invW : 0.f;
        sw2[e] = w2[e];
    }
    for (int e = t; e < 9 * C; e += 128) sw3[e] = w3[e];
    for (int e = t; e < C; e += 128) sb2[e] = b2[e];
    __syncthreads();
    int w = blockIdx.x * 128 + t;
    if (w >= W) return;
    int k0 = max(0, 5 - h), k1 = min(11, H + 5 - h);   // taps whose row lies inside the image
    float logit[9];
#pragma unroll
    for (int j = 0; j < 9; ++j) logit[j] = b3[j];
    for (int c = 0; c < C; ++c) {
        float a = A[((size_t)b * C + c) * W + w], s = Sm[(size_t)c * W + w];
        float v = sb2[c];
        for (int k = k0; k < k1; ++k) v = fmaf(sw2[c * 11 + k], fmaxf(fmaf(rm[k * C + c], s, a), 0.f), v);
#pragma unroll
        for (int j = 0; j < 9; ++j) logit[j] = fmaf(sw3[j * C + c], v, logit[j]);
    }
    size_t o = (((size_t)b * H + h) * W + w) * 9;
#pragma unroll
    for (int j = 0; j < 9; ++j) store_mixed<T>(mask, o + j, mask_f32, sigmoidf_(logit[j]));
}

// ------------------------------------------------------------------------------ SE
__global__ void se_excite_kernel(const float* __restrict__ gap_partial, int tiles, float inv_count,
                                 const float* __restrict__ w1, const float* __restrict__ b1,
                                 const float* __restrict__ w2, const float* __restrict__ b2,
                                 float* __restrict__ att, int C, int Hd) {
    extern __shared__ float sm[];
    float* mean = sm;        // [C]
    float* hid = sm + C;     // [Hd]
    int b = blockIdx.x, t = threadIdx.x;
    for (int c = t; c < C; c += blockDim.x) {
        float s = 0.f;
        for (int i = 0; i < tiles; ++i) s += gap_partial[((size_t)b * tiles + i) * C + c];
        mean[c] = s * inv_count;
    }
    __syncthreads();
    for (int h = t; h < Hd; h += blockDim.x) {
        float s = b1[h];
        for (int c = 0; c < C; ++c) s = fmaf(w1[(size_t)h * C + c], mean[c], s);
        hid[h] = fmaxf(s, 0.f);
    }
    __syncthreads();
    for (int c = t; c < C; c += blockDim.x) {
        float s = b2[c];
        for (int h = 0; h < Hd; ++h) s = fmaf(w2[(size_t)c * Hd + h], hid[h], s);
        att[(size_t)b * C + c] = sigmoidf_(s);
    }
}

constexpr int SQ_PIX = 256;   // pixels per squeeze tile

// grid (tiles, B), 256 threads: thread = (pixel lane, 8-channel vector) when C % 8 == 0 and 16-bit.
template <typename T>
__global__ void se_squeeze_kernel(const T* __restrict__ x, float* __restrict__ gap_partial, int HW, int C) {
    extern __shared__ float sm[];   // [rows][C]
    int b = blockIdx.y, tile = blockIdx.x, t = threadIdx.x;
    int p0 = tile * SQ_PIX, p1 = min(HW, p0 + SQ_PIX);
    int nC = min(C, 256), rows = 256 / nC;
    const T* xb = x + (size_t)b * HW * C;
    for (int cb = 0; cb < C; cb += nC) {
        int cl = t % nC, r = t / nC, c = cb + cl;
        float acc = 0.f;
        if (r < rows && c < C)
            for (int p = p0 + r; p < p1; p += rows) acc += to_f<T>(xb[(size_t)p * C + c]);
        sm[t] = acc;
        __syncthreads();
        if (t < nC && c < C) {
            float s = 0.f;
            for (int l = 0; l < rows; ++l) s += sm[l * nC + t];
            gap_partial[((size_t)b * gridDim.x + tile) * C + c] = s;
        }
        __syncthreads();
    }
}

template <typename T>
__global__ void se_rescale_kernel(const T* __restrict__ x, const float* __restrict__ att, T* __restrict__ y,
                                  size_t n, int HWC, int C) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        int b = (int)(e / HWC), c = (int)(e % C);
        y[e] = from_f<T>(to_f<T>(x[e]) * att[(size_t)b * C + c]);
    }
}

// 8 x 16-bit elements per thread (C % 8 == 0).
template <typename T>
__global__ void se_rescale_vec8_kernel(const uint4* __restrict__ x, const float* __restrict__ att,
                                       uint4* __restrict__ y, size_t nvec, int HWC8, int C8) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < nvec; e += (size_t)gridDim.x * blockDim.x) {
        int b = (int)(e / HWC8), c8 = (int)(e % C8);
        uint4 v = x[e];
        const float4* ap = reinterpret_cast<const float4*>(att + ((size_t)b * C8 + c8) * 8);
        float4 a0 = ap[0], a1 = ap[1];
        T* h = reinterpret_cast<T*>(&v);
        h[0] = from_f<T>(to_f<T>(h[0]) * a0.x); h[1] = from_f<T>(to_f<T>(h[1]) * a0.y);
        h[2] = from_f<T>(to_f<T>(h[2]) * a0.z); h[3] = from_f<T>(to_f<T>(h[3]) * a0.w);
        h[4] = from_f<T>(to_f<T>(h[4]) * a1.x); h[5] = from_f<T>(to_f<T>(h[5]) * a1.y);
        h[6] = from_f<T>(to_f<T>(h[6]) * a1.z); h[7] = from_f<T>(to_f<T>(h[7]) * a1.w);
        y[e] = v;
    }
}

// ------------------------------------------------------------------------------ KAD-Conv tail
struct MergeParams {
    const void* y[3]; const float* att[3];
    int c[3], h[3], w[3];
    float sy[3], sx[3];
    int H, W, C;
};

// Source index of bilinear resize with align_corners = False (half-pixel centres, clamped at 0).
__device__ __forceinline__ void src_index(int d, float scale, int in, int& i0, int& i1, float& l1) {
    float s = fmaxf(((float)d + 0.5f) * scale - 0.5f, 0.f);
    i0 = min((int)s, in - 1);
    i1 = i0 + (i0 < in - 1 ? 1 : 0);
    l1 = s - (float)i0;
}

template <typename T>
__global__ void merge_kernel(const T* __restrict__ x, T* __restrict__ out, MergeParams p, size_t n) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        int c = (int)(e % p.C);
        size_t pix = e / p.C;
        int xw = (int)(pix % p.W);
        size_t r = pix / p.W;
        int yh = (int)(r % p.H), b = (int)(r / p.H);
        int i = 0, cl = c;
        if (cl >= p.c[0]) { cl -= p.c[0]; i = 1; if (cl >= p.c[1]) { cl -= p.c[1]; i = 2; } }
        const T* yi = reinterpret_cast<const T*>(p.y[i]);
        int ci = p.c[i], hi = p.h[i], wi = p.w[i];
        float a = p.att[i][(size_t)b * ci + cl];
        float v;
        if (hi == p.H && wi == p.W) {
            v = to_f<T>(yi[(((size_t)b * hi + yh) * wi + xw) * ci + cl]);
        } else {
            int y0, y1, x0, x1; float ly, lx;
            src_index(yh, p.sy[i], hi, y0, y1, ly);
            src_index(xw, p.sx[i], wi, x0, x1, lx);
            const T* base = yi + (size_t)b * hi * wi * ci + cl;
            float v00 = to_f<T>(base[((size_t)y0 * wi + x0) * ci]), v01 = to_f<T>(base[((size_t)y0 * wi + x1) * ci]);
            float v10 = to_f<T>(base[((size_t)y1 * wi + x0) * ci]), v11 = to_f<T>(base[((size_t)y1 * wi + x1) * ci]);
            v = (1.f - ly) * ((1.f - lx) * v00 + lx * v01) + ly * ((1.f - lx) * v10 + lx * v11);
        }
        out[e] = from_f<T>(fmaf(v, a, to_f<T>(x[e])));
    }
}

inline int grid_for(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    size_t cap = 148 * 16;
    return (int)(g < cap ? (g ? g : 1) : cap);
}

template <typename T>
int launch_transpose(const void* src, void* dst, int B, int R, int S, cudaStream_t st) {
    dim3 grid((S + 31) / 32, (R + 31) / 32, B), block(32, 8);
    transpose_kernel<T><<<grid, block, 0, st>>>((const T*)src, (T*)dst, R, S);
    return 0;
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" int kad_nchw_to_nhwc(const void* src, void* dst, int B, int C, int H, int W, int dtype, void* stream) {
    KAD_CHECK_ARG(src && dst && B > 0 && C > 0 && H > 0 && W > 0, "kad_nchw_to_nhwc: bad argument");
    KAD_CHECK_ARG(B <= 65535, "kad_nchw_to_nhwc: batch %d too large", B);
    if (dtype == KAD_F32) launch_transpose<float>(src, dst, B, C, H * W, (cudaStream_t)stream);
    else if (dtype == KAD_F16 || dtype == KAD_BF16) launch_transpose<uint16_t>(src, dst, B, C, H * W, (cudaStream_t)stream);
    else return fail(KAD_ERR_INVALID, "unknown dtype %d", dtype);
    KAD_CHECK_LAUNCH("transpose_kernel");
    return KAD_OK;
}

extern "C" int kad_nhwc_to_nchw(const void* src, void* dst, int B, int C, int H, int W, int dtype, void* stream) {
    KAD_CHECK_ARG(src && dst && B > 0 && C > 0 && H > 0 && W > 0, "kad_nhwc_to_nchw: bad argument");
    KAD_CHECK_ARG(B <= 65535, "kad_nhwc_to_nchw: batch %d too large", B);
    if (dtype == KAD_F32) launch_transpose<float>(src, dst, B, H * W, C, (cudaStream_t)stream);
    else if (dtype == KAD_F16 || dtype == KAD_BF16) launch_transpose<uint16_t>(src, dst, B, H * W, C, (cudaStream_t)stream);
    else return fail(KAD_ERR_INVALID, "unknown dtype %d", dtype);
    KAD_CHECK_LAUNCH("transpose_kernel");
    return KAD_OK;
}

extern "C" int kad_lcsa_sums(const void* x, float* rowsum, float* colsum, int B, int H, int W, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(x && rowsum && colsum && B > 0 && H > 0 && W > 0 && C > 0, "kad_lcsa_sums: bad argument");
    KAD_CHECK_ARG(B <= 65535, "kad_lcsa_sums: batch %d too large", B);
    cudaStream_t st = (cudaStream_t)stream;
    KAD_DISPATCH_DTYPE(dtype, {
        lcsa_rowsum_kernel<T><<<dim3(H, B), 256, 0, st>>>((const T*)x, rowsum, H, W, C);
        lcsa_colsum_kernel<T><<<dim3((W * C + 255) / 256, B), 256, 0, st>>>((const T*)x, colsum, H, W, C);
    });
    KAD_CHECK_LAUNCH("lcsa_sums");
    return KAD_OK;
}

extern "C" int kad_lcsa_mask(const float* rowsum, const float* colsum,
                             const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                             const float* w2, const float* b2, const float* w3, const float* b3,
                             float* scratch, void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream) {
    KAD_CHECK_ARG(rowsum && colsum && w1 && b1 && bn_scale && bn_shift && w2 && b2 && w3 && b3 && scratch && mask,
                  "kad_lcsa_mask: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && C > 0 && B <= 65535 && H <= 65535, "kad_lcsa_mask: bad shape");
    size_t smem = sizeof(float) * (size_t)(11 + 11 + 9 + 1) * C;
    KAD_CHECK_ARG(smem <= 200 * 1024, "kad_lcsa_mask: %d channels exceed the shared-memory staging", C);
    cudaStream_t st = (cudaStream_t)stream;
    float* A = scratch;
    float* Sm = scratch + (size_t)B * W * C;
    lcsa_prep_kernel<<<dim3((W * C + 255) / 256, B), 256, 0, st>>>(colsum, w1, b1, bn_scale, bn_shift, A, Sm, H, W, C);
    KAD_DISPATCH_DTYPE(dtype, {
        auto kern = lcsa_mask_kernel<T>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "lcsa_mask smem attribute: %s", cudaGetErrorString(e));
        }
        kern<<<dim3((W + 127) / 128, H, B), 128, smem, st>>>(rowsum, A, Sm, w2, b2, w3, b3, mask, H, W, C, mask_f32);
    });
    KAD_CHECK_LAUNCH("lcsa_mask");
    return KAD_OK;
}

extern "C" int kad_se_excite(const float* gap_partial, int tiles, float inv_count,
                             const float* w1, const float* b1, const float* w2, const float* b2,
                             float* att, int B, int C, int Hd, void* stream) {
    KAD_CHECK_ARG(gap_partial && w1 && b1 && w2 && b2 && att, "kad_se_excite: null pointer");
    KAD_CHECK_ARG(B > 0 && C > 0 && Hd > 0 && tiles > 0, "kad_se_excite: bad shape");
    size_t smem = sizeof(float) * (size_t)(C + Hd);
    KAD_CHECK_ARG(smem <= 48 * 1024, "kad_se_excite: C + hidden = %d too large", C + Hd);
    se_excite_kernel<<<B, 256, smem, (cudaStream_t)stream>>>(gap_partial, tiles, inv_count, w1, b1, w2, b2, att, C, Hd);
    KAD_CHECK_LAUNCH("se_excite_kernel");
    return KAD_OK;
}

extern "C" int kad_se_squeeze_tiles(int H, int W) { return (H * W + SQ_PIX - 1) / SQ_PIX; }

extern "C" int kad_se_squeeze(const void* x, float* gap_partial, int B, int H, int W, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(x && gap_partial && B > 0 && H > 0 && W > 0 && C > 0 && B <= 65535, "kad_se_squeeze: bad argument");
    dim3 grid(kad_se_squeeze_tiles(H, W), B);
    KAD_DISPATCH_DTYPE(dtype, {
        se_squeeze_kernel<T><<<grid, 256, 256 * sizeof(float), (cudaStream_t)stream>>>((const T*)x, gap_partial, H * W, C);
    });
    KAD_CHECK_LAUNCH("se_squeeze_kernel");
    return KAD_OK;
}

extern "C" int kad_se_rescale(const void* x, const float* att, void* y, int B, int H, int W, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(x && att && y && B > 0 && H > 0 && W > 0 && C > 0, "kad_se_rescale: bad argument");
    size_t n = (size_t)B * H * W * C;
    cudaStream_t st = (cudaStream_t)stream;
    bool vec = dtype != KAD_F32 && C % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && ((uintptr_t)att % 16 == 0);
    if (vec) {
        size_t nv = n / 8;
        if (dtype == KAD_F16)
            se_rescale_vec8_kernel<__half><<<grid_for(nv, 256), 256, 0, st>>>((const uint4*)x, att, (uint4*)y, nv, H * W * C / 8, C / 8);
        else
            se_rescale_vec8_kernel<__nv_bfloat16><<<grid_for(nv, 256), 256, 0, st>>>((const uint4*)x, att, (uint4*)y, nv, H * W * C / 8, C / 8);
    } else {
        KAD_DISPATCH_DTYPE(dtype, {
            se_rescale_kernel<T><<<grid_for(n, 256), 256, 0, st>>>((const T*)x, att, (T*)y, n, H * W * C, C);
        });
    }
    KAD_CHECK_LAUNCH("se_rescale_kernel");
    return KAD_OK;
}

extern "C" int kad_merge_upsample_residual(const KadMergeArgs* a, void* stream) {
    KAD_CHECK_ARG(a && a->x && a->out, "kad_merge_upsample_residual: null pointer");
    KAD_CHECK_ARG(a->B > 0 && a->H > 0 && a->W > 0 && a->C > 0, "kad_merge_upsample_residual: bad shape");
    KAD_CHECK_ARG(a->c[0] + a->c[1] + a->c[2] == a->C, "kad_merge_upsample_residual: branch widths %d+%d+%d != %d",
                  a->c[0], a->c[1], a->c[2], a->C);
    MergeParams p;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(a->y[i] && a->att[i] && a->h[i] > 0 && a->w[i] > 0, "kad_merge_upsample_residual: bad branch %d", i);
        p.y[i] = a->y[i]; p.att[i] = a->att[i]; p.c[i] = a->c[i]; p.h[i] = a->h[i]; p.w[i] = a->w[i];
        p.sy[i] = (float)a->h[i] / (float)a->H; p.sx[i] = (float)a->w[i] / (float)a->W;
    }
    p.H = a->H; p.W = a->W; p.C = a->C;
    size_t n = (size_t)a->B * a->H * a->W * a->C;
    KAD_DISPATCH_DTYPE(a->dtype, {
        merge_kernel<T><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const T*)a->x, (T*)a->out, p, n);
    });
    KAD_CHECK_LAUNCH("merge_kernel");
    return KAD_OK;
}


// ------------------------------------------------------------------------------ allocation-free LCSA mask
// Some hosts of this library may not create device memory on their frame path: an inference server that handed
// the whole HBM to its own pool at start-up has nothing left for cudaMalloc to return, and a latency-bound loop
// cannot afford the device-wide synchronisation that cudaMalloc / cudaFree imply. kad_lcsa_mask() asks such a
// caller for a scratch buffer it may not be able to produce; this variant keeps the scratch inside the library
// image instead: a fixed array in device memory that every GPU loading the library holds until the process exits.
namespace {
constexpr size_t LCSA_STATIC_FLOATS = (size_t)1 << 20;                 // 4 MiB of float32 per device
static __device__ __align__(256) float g_lcsa_scratch[LCSA_STATIC_FLOATS];
constexpr int MAX_DEVICES = 64;
float* g_lcsa_scratch_ptr[MAX_DEVICES] = {};                           // device address of the array, per device
std::mutex g_lcsa_scratch_mutex;
}  // namespace

extern "C" size_t kad_lcsa_mask_noalloc_max_floats(void) { return LCSA_STATIC_FLOATS; }

extern "C" int kad_lcsa_mask_noalloc(const float* rowsum, const float* colsum,
                                     const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                                     const float* w2, const float* b2, const float* w3, const float* b3,
                                     void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream) {
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && C > 0, "kad_lcsa_mask_noalloc: bad shape");
    const size_t need = ((size_t)B + 1) * (size_t)W * (size_t)C;
    if (need > LCSA_STATIC_FLOATS)
        return fail(KAD_ERR_UNSUPPORTED, "kad_lcsa_mask_noalloc: (B+1)*W*C = %zu floats exceeds the built-in scratch of %zu floats; "
                    "use kad_lcsa_mask with a caller-provided scratch buffer", need, (size_t)LCSA_STATIC_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_lcsa_mask_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    KAD_CHECK_ARG(dev >= 0 && dev < MAX_DEVICES, "kad_lcsa_mask_noalloc: device index %d out of range", dev);
    float* scratch = nullptr;
    {
        // First call on this device: resolve the array's DEVICE address. In host code the symbol itself is only a
        // host-side handle, not something a kernel can dereference, so the address must come from the runtime,
        // queried while this device is current.
        std::lock_guard<std::mutex> lock(g_lcsa_scratch_mutex);
        if (!g_lcsa_scratch_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_lcsa_scratch);
            if (e != cudaSuccess || !p)
                return fail(KAD_ERR_CUDA, "kad_lcsa_mask_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_lcsa_scratch_ptr[dev] = static_cast<float*>(p);
        }
        scratch = g_lcsa_scratch_ptr[dev];
    }
    // Every element of scratch[0, need) is overwritten before it is read, so stale contents of an earlier call are harmless.
    return kad_lcsa_mask(rowsum, colsum, w1, b1, bn_scale, bn_shift, w2, b2, w3, b3, scratch, mask, B, H, W, C, mask_f32, dtype, stream);
}
