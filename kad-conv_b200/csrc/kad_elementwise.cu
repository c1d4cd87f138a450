// Bandwidth-bound kernels of the KAD-Conv path: layout conversion, the LCSA mask branch, the SE
// squeeze / excite / rescale, and the upsample + concat + residual tail. All NHWC, fp32 arithmetic.
#include <mutex>

#include "kad_mma.cuh"

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

// grid (ceil(W/128), H, B), 128 threads; each thread one pixel. Per channel the 11 row means, the 11 vertical taps
// and the 9 projection weights are staged as padded rows of 12 floats, so the inner loop reads 9 broadcast float4s.
template <typename T>
__global__ void __launch_bounds__(128)
lcsa_mask_kernel(const float* __restrict__ rowsum, const float* __restrict__ A, const float* __restrict__ Sm,
                 const float* __restrict__ w2, const float* __restrict__ b2, const float* __restrict__ w3,
                 const float* __restrict__ b3, void* __restrict__ mask, int H, int W, int C, int mask_f32) {
    extern __shared__ __align__(16) float sm[];
    float* rm = sm;               // [C][12] row means of rows h-5..h+5 (0 outside the image), pad 0
    float* sw2 = rm + 12 * C;     // [C][12] 11x1 taps (0 for rows outside the image), slot 11 = bias b2
    float* sw3 = sw2 + 12 * C;    // [C][12] 1x1 weights of the 9 outputs, pad 0
    int b = blockIdx.z, h = blockIdx.y, t = threadIdx.x;
    float invW = 1.f / (float)W;
    for (int e = t; e < 12 * C; e += 128) {
        int c = e / 12, k = e - c * 12, hh = h + k - 5;
        bool in = k < 11 && hh >= 0 && hh < H;
        rm[e] = in ? rowsum[((size_t)b * H + hh) * C + c] * invW : 0.f;
        sw2[e] = in ? w2[c * 11 + k] : (k == 11 ? b2[c] : 0.f);
        sw3[e] = k < 9 ? w3[k * C + c] : 0.f;
    }
    __syncthreads();
    int w = blockIdx.x * 128 + t;
    if (w >= W) return;
    float logit[9];
#pragma unroll
    for (int j = 0; j < 9; ++j) logit[j] = b3[j];
    const float4* rm4 = reinterpret_cast<const float4*>(rm);
    const float4* w24 = reinterpret_cast<const float4*>(sw2);
    const float4* w34 = reinterpret_cast<const float4*>(sw3);
    for (int c = 0; c < C; ++c) {
        const float a = A[((size_t)b * C + c) * W + w], s = Sm[(size_t)c * W + w];
        const float4 r0 = rm4[3 * c], r1 = rm4[3 * c + 1], r2 = rm4[3 * c + 2];
        const float4 u0 = w24[3 * c], u1 = w24[3 * c + 1], u2 = w24[3 * c + 2];
        float v = u2.w;           // bias of the 11x1 convolution
        v = fmaf(u0.x, fmaxf(fmaf(r0.x, s, a), 0.f), v); v = fmaf(u0.y, fmaxf(fmaf(r0.y, s, a), 0.f), v);
        v = fmaf(u0.z, fmaxf(fmaf(r0.z, s, a), 0.f), v); v = fmaf(u0.w, fmaxf(fmaf(r0.w, s, a), 0.f), v);
        v = fmaf(u1.x, fmaxf(fmaf(r1.x, s, a), 0.f), v); v = fmaf(u1.y, fmaxf(fmaf(r1.y, s, a), 0.f), v);
        v = fmaf(u1.z, fmaxf(fmaf(r1.z, s, a), 0.f), v); v = fmaf(u1.w, fmaxf(fmaf(r1.w, s, a), 0.f), v);
        v = fmaf(u2.x, fmaxf(fmaf(r2.x, s, a), 0.f), v); v = fmaf(u2.y, fmaxf(fmaf(r2.y, s, a), 0.f), v);
        v = fmaf(u2.z, fmaxf(fmaf(r2.z, s, a), 0.f), v);
        const float4 p0 = w34[3 * c], p1 = w34[3 * c + 1], p2 = w34[3 * c + 2];
        logit[0] = fmaf(p0.x, v, logit[0]); logit[1] = fmaf(p0.y, v, logit[1]); logit[2] = fmaf(p0.z, v, logit[2]);
        logit[3] = fmaf(p0.w, v, logit[3]); logit[4] = fmaf(p1.x, v, logit[4]); logit[5] = fmaf(p1.y, v, logit[5]);
        logit[6] = fmaf(p1.z, v, logit[6]); logit[7] = fmaf(p1.w, v, logit[7]); logit[8] = fmaf(p2.x, v, logit[8]);
    }
    size_t o = (((size_t)b * H + h) * W + w) * 9;
#pragma unroll
    for (int j = 0; j < 9; ++j) store_mixed<T>(mask, o + j, mask_f32, sigmoid_mask(logit[j]));
}

// ---- LCSA from the partial sums the pyramid kernel leaves behind --------------------------------------------------------
// grid (ceil(W / 16), B): a block finishes the column sums of its 16 columns and of the 5 neighbours on either side (the
// reach of the 1x11 convolution) in shared memory, then A and Sm of its columns as in lcsa_prep_kernel; the blocks of an
// image also share out its rows for the row sums. Fixed summation order.
constexpr int PREP_COLS = 16;
__global__ void __launch_bounds__(256)
lcsa_prep_partials_kernel(const float* __restrict__ rowpart, int nct, const float* __restrict__ colpart, int nrg,
                          const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ bn_m,
                          const float* __restrict__ bn_a, float* __restrict__ A, float* __restrict__ Sm, float* __restrict__ rowsum,
                          int H, int W, int C, int Cp) {
    // A [B][W][Cp], Sm [W][Cp] (channels innermost, padded to a multiple of 4: the mask kernel reads them as float4)
    extern __shared__ float colsum_s[];          // [PREP_COLS + 10][C], column w0 - 5 first
    grid_dependency_wait();                      // everything here reads the partial sums of the kernel before
    grid_dependents_go();
    const int b = blockIdx.y, t = threadIdx.x;
    const int w0 = blockIdx.x * PREP_COLS, nw = min(PREP_COLS, W - w0);
    const int lo = max(0, w0 - 5), hi = min(W, w0 + nw + 5);      // columns [lo, hi) are summed
    const float* cp = colpart + (size_t)b * nrg * W * C;
    for (int e = t; e < (hi - lo) * C; e += 256) {
        float s = 0.f;
#pragma unroll 4
        for (int g = 0; g < nrg; ++g) s += cp[((size_t)g * W + lo) * C + e];
        colsum_s[(lo - (w0 - 5)) * C + e] = s;
    }
    // rows of this image handled by this block
    const int rows_per = (H + gridDim.x - 1) / gridDim.x, h0 = blockIdx.x * rows_per, h1 = min(H, h0 + rows_per);
    for (int e = t; e < (h1 - h0) * C; e += 256) {
        const int h = h0 + e / C, c = e % C;
        float s = 0.f;
#pragma unroll 4
        for (int k = 0; k < nct; ++k) s += rowpart[(((size_t)b * H + h) * nct + k) * C + c];
        rowsum[((size_t)b * H + h) * C + c] = s;
    }
    __syncthreads();
    const float invH = 1.f / (float)H;
    for (int e = t; e < nw * Cp; e += 256) {
        const int wl = e / Cp, c = e - wl * Cp, w = w0 + wl;
        float av = 0.f, sv = 0.f;
        if (c < C) {
            float conv = 0.f, S = 0.f;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const int ww = w + k - 5;
                if (ww >= 0 && ww < W) {
                    const float wk = w1[c * 11 + k];
                    conv = fmaf(wk, colsum_s[(ww - (w0 - 5)) * C + c] * invH, conv);
                    S += wk;
                }
            }
            const float m = bn_m[c];
            av = (conv + b1[c]) * m + bn_a[c]; sv = S * m;
        }
        A[((size_t)b * W + w) * Cp + c] = av;
        if (b == 0) Sm[(size_t)w * Cp + c] = sv;
    }
}

// n floats staged in shared memory in the order they have in global memory (they go to g[o0 .. o0 + n)), written with 16-byte
// stores. A thread that owns a pixel would store its nine masks 36 bytes apart from its neighbour's: nine store instructions per
// warp that each touch 36 sectors partially. `stage` holds element i at stage[(o0 & 3) + i], so that the 16-byte groups of shared
// and global memory coincide whatever the offset of the block's first element (g itself is 16-byte aligned).
__device__ __forceinline__ void store_staged_f32(float* __restrict__ g, size_t o0, const float* __restrict__ stage, int n, int t, int nthreads) {
    const int mis = (int)(o0 & 3), head = mis ? min(n, 4 - mis) : 0;
    if (t < head) g[o0 + t] = stage[mis + t];
    const int nb = (n - head) >> 2;
    const float4* s4 = reinterpret_cast<const float4*>(stage + mis + head);
    float4* g4 = reinterpret_cast<float4*>(g + o0 + head);
    for (int k = t; k < nb; k += nthreads) g4[k] = s4[k];
    const int done = head + 4 * nb;
    if (t < n - done) g[o0 + done + t] = stage[mis + done + t];
}

// The mask for 128 CONSECUTIVE pixels of an image per block (so narrow feature maps do not leave most lanes idle): the
// staged operands of lcsa_mask_kernel, once per image row the block touches.
template <typename T>
__global__ void __launch_bounds__(128)
lcsa_mask_flat_kernel(const float* __restrict__ rowsum, const float* __restrict__ A, const float* __restrict__ Sm,
                      const float* __restrict__ w2, const float* __restrict__ b2, const float* __restrict__ w3,
                      const float* __restrict__ b3, void* __restrict__ mask, int H, int W, int C, int Cp, int mask_f32, int rows_are_means, int staged) {
    extern __shared__ __align__(16) float sm[];
    const int b = blockIdx.y, t = threadIdx.x, HW = H * W;
    const int p0 = blockIdx.x * 128, p1 = min(HW, p0 + 128);
    const int r_lo = p0 / W, nrows = (p1 - 1) / W - r_lo + 1;
    float* sw3 = sm;                     // [Cp][12] 1x1 weights of the 9 outputs, pad 0
    float* rm = sw3 + 12 * Cp;           // [nrows][Cp][12] row means of rows h-5..h+5 (0 outside the image), pad 0
    float* sw2 = rm + nrows * 12 * Cp;   // [nrows][Cp][12] 11x1 taps (0 for rows outside the image), slot 11 = bias b2
    float* stage = sw2 + nrows * 12 * Cp;     // [3 + 128 * 9] the block's masks in global order (only with `staged`)
    const float invW = rows_are_means ? 1.f : 1.f / (float)W;      // `rowsum` holds row means already
    for (int e = t; e < 12 * Cp; e += 128) { const int c = e / 12, k = e - c * 12; sw3[e] = (k < 9 && c < C) ? w3[k * C + c] : 0.f; }
    grid_dependency_wait();              // the weights above are parameters; rowsum, A and Sm come from the kernel before
    grid_dependents_go();
    for (int e = t; e < nrows * 12 * Cp; e += 128) {
        const int r = e / (12 * Cp), rem = e - r * 12 * Cp, c = rem / 12, k = rem - c * 12, hh = r_lo + r + k - 5;
        const bool in = k < 11 && hh >= 0 && hh < H && c < C;
        rm[e] = in ? rowsum[((size_t)b * H + hh) * C + c] * invW : 0.f;
        sw2[e] = in ? w2[c * 11 + k] : ((k == 11 && c < C) ? b2[c] : 0.f);
    }
    __syncthreads();
    const int p = p0 + t;
    const size_t o0 = ((size_t)b * HW + p0) * 9;
    if (p < HW) {
    const int h = p / W, w = p - h * W, r = h - r_lo;
    float logit[9];
#pragma unroll
    for (int j = 0; j < 9; ++j) logit[j] = b3[j];
    const float4* rm4 = reinterpret_cast<const float4*>(rm + (size_t)r * 12 * Cp);
    const float4* w24 = reinterpret_cast<const float4*>(sw2 + (size_t)r * 12 * Cp);
    const float4* w34 = reinterpret_cast<const float4*>(sw3);
    // this pixel's column terms for all channels: contiguous, read four channels at a time (no dependent load per channel)
    const float4* A4 = reinterpret_cast<const float4*>(A + ((size_t)b * W + w) * Cp);
    const float4* S4 = reinterpret_cast<const float4*>(Sm + (size_t)w * Cp);
#pragma unroll 2
    for (int c4 = 0; c4 < (Cp >> 2); ++c4) {
        const float4 av = __ldg(A4 + c4), sv = __ldg(S4 + c4);
        const float aa[4] = {av.x, av.y, av.z, av.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const int c = 4 * c4 + j4;
            const float a = aa[j4], s = ss[j4];
            const float4 r0 = rm4[3 * c], r1 = rm4[3 * c + 1], r2 = rm4[3 * c + 2];
            const float4 u0 = w24[3 * c], u1 = w24[3 * c + 1], u2 = w24[3 * c + 2];
            float v = u2.w;           // bias of the 11x1 convolution (0 for a padding channel, whose weights are 0 as well)
            v = fmaf(u0.x, fmaxf(fmaf(r0.x, s, a), 0.f), v); v = fmaf(u0.y, fmaxf(fmaf(r0.y, s, a), 0.f), v);
            v = fmaf(u0.z, fmaxf(fmaf(r0.z, s, a), 0.f), v); v = fmaf(u0.w, fmaxf(fmaf(r0.w, s, a), 0.f), v);
            v = fmaf(u1.x, fmaxf(fmaf(r1.x, s, a), 0.f), v); v = fmaf(u1.y, fmaxf(fmaf(r1.y, s, a), 0.f), v);
            v = fmaf(u1.z, fmaxf(fmaf(r1.z, s, a), 0.f), v); v = fmaf(u1.w, fmaxf(fmaf(r1.w, s, a), 0.f), v);
            v = fmaf(u2.x, fmaxf(fmaf(r2.x, s, a), 0.f), v); v = fmaf(u2.y, fmaxf(fmaf(r2.y, s, a), 0.f), v);
            v = fmaf(u2.z, fmaxf(fmaf(r2.z, s, a), 0.f), v);
            const float4 q0 = w34[3 * c], q1 = w34[3 * c + 1], q2 = w34[3 * c + 2];
            logit[0] = fmaf(q0.x, v, logit[0]); logit[1] = fmaf(q0.y, v, logit[1]); logit[2] = fmaf(q0.z, v, logit[2]);
            logit[3] = fmaf(q0.w, v, logit[3]); logit[4] = fmaf(q1.x, v, logit[4]); logit[5] = fmaf(q1.y, v, logit[5]);
            logit[6] = fmaf(q1.z, v, logit[6]); logit[7] = fmaf(q1.w, v, logit[7]); logit[8] = fmaf(q2.x, v, logit[8]);
        }
    }
    if (staged) {
        float* so = stage + (int)(o0 & 3) + t * 9;
#pragma unroll
        for (int j = 0; j < 9; ++j) so[j] = sigmoid_mask(logit[j]);
    } else {
        const size_t o = o0 + (size_t)t * 9;
#pragma unroll
        for (int j = 0; j < 9; ++j) store_mixed<T>(mask, o + j, mask_f32, sigmoid_mask(logit[j]));
    }
    }
    if (staged) {                        // uniform over the block
        __syncthreads();
        store_staged_f32(reinterpret_cast<float*>(mask), o0, stage, (p1 - p0) * 9, t, 128);
    }
}

// The same mask for column strips: a thread owns LS_R vertically consecutive pixels of one column, so the ReLU'd
// intermediate t(h) = relu(rowmean(h) * S + A) of the LS_R + 10 rows its 11x1 windows cover is evaluated once and shared
// by the windows (2 * (LS_R + 10) instead of 22 * LS_R operations per channel), and the staged operands are read once
// per strip instead of once per pixel. A block covers all W <= 128 columns of groups * LS_R rows of one image.
constexpr int LS_R = 4;
template <typename T>
__global__ void __launch_bounds__(128)
lcsa_mask_strip_kernel(const float* __restrict__ rowsum, const float* __restrict__ A, const float* __restrict__ Sm,
                       const float* __restrict__ w2, const float* __restrict__ b2, const float* __restrict__ w3,
                       const float* __restrict__ b3, void* __restrict__ mask, int H, int W, int C, int Cp, int groups, int mask_f32, int rows_are_means, int staged) {
    extern __shared__ __align__(16) float sm[];
    const int b = blockIdx.y, t = threadIdx.x;
    const int RB = groups * LS_R, P = RB + 12;           // rows per block; row pitch of the staged means (rows h0-5 .. h0+RB+6)
    const int h0 = blockIdx.x * RB;
    float* sw3 = sm;                     // [Cp][12] 1x1 weights of the 9 outputs, pad 0
    float* sw2 = sw3 + 12 * Cp;          // [Cp][12] 11x1 taps, slot 11 = bias b2
    float* rm = sw2 + 12 * Cp;           // [Cp][P] row means (0 outside the image; those rows are masked below)
    float* stage = rm + Cp * P;          // [3 + RB * W * 9] the block's masks in global order (only with `staged`)
    const float invW = rows_are_means ? 1.f : 1.f / (float)W;
    for (int e = t; e < 12 * Cp; e += 128) {
        const int c = e / 12, k = e - c * 12;
        sw3[e] = (k < 9 && c < C) ? w3[k * C + c] : 0.f;
        sw2[e] = c < C ? (k < 11 ? w2[c * 11 + k] : b2[c]) : 0.f;
    }
    grid_dependency_wait();              // the weights above are parameters; rowsum, A and Sm come from the kernel before
    grid_dependents_go();
    for (int e = t; e < Cp * P; e += 128) {
        const int j = e / Cp, c = e - j * Cp, hh = h0 - 5 + j;       // consecutive threads read consecutive channels
        rm[c * P + j] = (hh >= 0 && hh < H && c < C) ? rowsum[((size_t)b * H + hh) * C + c] * invW : 0.f;
    }
    __syncthreads();
    const int g = t / W, w = t - g * W;
    const int r0 = h0 + g * LS_R;                        // first row of this thread's strip
    const size_t o0 = ((size_t)b * H + h0) * W * 9;      // the block's first mask element
    if (g < groups && r0 < H) {
    uint32_t valid = 0;                                  // bit j: row r0 - 5 + j lies inside the image
#pragma unroll
    for (int j = 0; j < LS_R + 10; ++j) valid |= (uint32_t)(r0 - 5 + j >= 0 && r0 - 5 + j < H) << j;
    float logit[LS_R][9];
#pragma unroll
    for (int r = 0; r < LS_R; ++r)
#pragma unroll
        for (int j = 0; j < 9; ++j) logit[r][j] = b3[j];
    const float4* A4 = reinterpret_cast<const float4*>(A + ((size_t)b * W + w) * Cp);
    const float4* S4 = reinterpret_cast<const float4*>(Sm + (size_t)w * Cp);
    const float4* w24 = reinterpret_cast<const float4*>(sw2);
    const float4* w34 = reinterpret_cast<const float4*>(sw3);
#pragma unroll 1
    for (int c4 = 0; c4 < (Cp >> 2); ++c4) {
        const float4 av = __ldg(A4 + c4), sv = __ldg(S4 + c4);
        const float aa[4] = {av.x, av.y, av.z, av.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const int c = 4 * c4 + j4;
            const float a = aa[j4], s = ss[j4];
            const float4* rm4 = reinterpret_cast<const float4*>(rm + c * P + g * LS_R);
            float tv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float4 v4 = rm4[q]; tv[4 * q] = v4.x; tv[4 * q + 1] = v4.y; tv[4 * q + 2] = v4.z; tv[4 * q + 3] = v4.w; }
#pragma unroll
            for (int j = 0; j < LS_R + 10; ++j) tv[j] = ((valid >> j) & 1u) ? fmaxf(fmaf(tv[j], s, a), 0.f) : 0.f;
            const float4 u0 = w24[3 * c], u1 = w24[3 * c + 1], u2 = w24[3 * c + 2];
            const float uk[11] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w, u2.x, u2.y, u2.z};
            const float4 q0 = w34[3 * c], q1 = w34[3 * c + 1], q2 = w34[3 * c + 2];
#pragma unroll
            for (int r = 0; r < LS_R; ++r) {
                float v = u2.w;       // bias of the 11x1 convolution (0 for a padding channel, whose weights are 0 as well)
#pragma unroll
                for (int k = 0; k < 11; ++k) v = fmaf(uk[k], tv[r + k], v);
                logit[r][0] = fmaf(q0.x, v, logit[r][0]); logit[r][1] = fmaf(q0.y, v, logit[r][1]); logit[r][2] = fmaf(q0.z, v, logit[r][2]);
                logit[r][3] = fmaf(q0.w, v, logit[r][3]); logit[r][4] = fmaf(q1.x, v, logit[r][4]); logit[r][5] = fmaf(q1.y, v, logit[r][5]);
                logit[r][6] = fmaf(q1.z, v, logit[r][6]); logit[r][7] = fmaf(q1.w, v, logit[r][7]); logit[r][8] = fmaf(q2.x, v, logit[r][8]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < LS_R; ++r) {
        if (r0 + r >= H) break;
        if (staged) {
            float* so = stage + (int)(o0 & 3) + ((g * LS_R + r) * W + w) * 9;
#pragma unroll
            for (int j = 0; j < 9; ++j) so[j] = sigmoid_mask(logit[r][j]);
        } else {
            const size_t o = ((size_t)b * H * W + (size_t)(r0 + r) * W + w) * 9;
#pragma unroll
            for (int j = 0; j < 9; ++j) store_mixed<T>(mask, o + j, mask_f32, sigmoid_mask(logit[r][j]));
        }
    }
    }
    if (staged) {                        // uniform over the block
        __syncthreads();
        store_staged_f32(reinterpret_cast<float*>(mask), o0, stage, min(RB, H - h0) * W * 9, t, 128);
    }
}

// ---- the three LCSA masks of a KAD-Conv layer in ONE launch, straight from the pyramid kernel's partial sums -------------------
// What lcsa_prep_partials_kernel + lcsa_mask_strip_kernel / lcsa_mask_flat_kernel do in two launches per branch (six per layer):
// a block first finishes, in shared memory, the first stage of ITS branch and image for the columns and rows it needs (column sums
// over the row groups, the separable 1x11 convolution + BatchNorm -> A and Sm for every column; row means of its rows and the five
// above and below), then evaluates the masks of its rows as column strips of LS_R rows per thread (lcsa_mask_strip_kernel's
// arithmetic, in the same order: the results are bit-identical to the two-launch path). The first stage is recomputed by every
// block of an image (a few thousand L2 loads and FMAs against ~100 k FMAs of mask work per block); in exchange the layer's
// LCSAs are one graph node in front of the fork instead of six on the branch streams.
struct LcsaBranch {
    const float* rowpart; const float* colpart;
    const float* w1; const float* b1; const float* bn_m; const float* bn_a; const float* w2; const float* b2; const float* w3; const float* b3;
    void* mask;
    int H, W, C, Cp, groups, row_blocks, first_block;
};
struct LcsaFusedParams { LcsaBranch br[3]; int nct, nrg, mask_f32; };

template <typename T>
__global__ void __launch_bounds__(128)
lcsa_fused_kernel(const LcsaFusedParams p) {
    extern __shared__ __align__(16) float sm[];
    const int t = threadIdx.x, b = blockIdx.y;
    const int i = (int)blockIdx.x >= p.br[2].first_block ? 2 : ((int)blockIdx.x >= p.br[1].first_block ? 1 : 0);
    const LcsaBranch& q = i == 0 ? p.br[0] : (i == 1 ? p.br[1] : p.br[2]);
    const int H = q.H, W = q.W, C = q.C, Cp = q.Cp, groups = q.groups;
    const int RB = groups * LS_R, P = RB + 12;           // rows per block; row pitch of the staged means (rows h0-5 .. h0+RB+6)
    const int h0 = ((int)blockIdx.x - q.first_block) * RB;
    float* sw3 = sm;                     // [Cp][12] 1x1 weights of the 9 outputs, pad 0
    float* sw2 = sw3 + 12 * Cp;          // [Cp][12] 11x1 taps, slot 11 = bias b2
    float* rm = sw2 + 12 * Cp;           // [Cp][P] row means (0 outside the image; those rows are masked below)
    float* As = rm + Cp * P;             // [W][Cp]
    float* Sms = As + W * Cp;            // [W][Cp]
    float* colsum_s = Sms + W * Cp;      // [W][C]
    // ---- first stage ------------------------------------------------------------------------------------------------------
    const float* cp = q.colpart + (size_t)b * p.nrg * W * C;
    for (int e = t; e < W * C; e += 128) {
        float s = 0.f;
#pragma unroll 4
        for (int g = 0; g < p.nrg; ++g) s += cp[(size_t)g * W * C + e];
        colsum_s[e] = s;
    }
    for (int e = t; e < 12 * Cp; e += 128) {
        const int c = e / 12, k = e - c * 12;
        sw3[e] = (k < 9 && c < C) ? q.w3[k * C + c] : 0.f;
        sw2[e] = c < C ? (k < 11 ? q.w2[c * 11 + k] : q.b2[c]) : 0.f;
    }
    const float invW = 1.f / (float)W;
    for (int e = t; e < Cp * P; e += 128) {
        const int j = e / Cp, c = e - j * Cp, hh = h0 - 5 + j;       // consecutive threads read consecutive channels
        float v = 0.f;
        if (hh >= 0 && hh < H && c < C) {
            float s = 0.f;
#pragma unroll 4
            for (int k = 0; k < p.nct; ++k) s += q.rowpart[(((size_t)b * H + hh) * p.nct + k) * C + c];
            v = s * invW;
        }
        rm[c * P + j] = v;
    }
    __syncthreads();
    const float invH = 1.f / (float)H;
    for (int e = t; e < W * Cp; e += 128) {
        const int w = e / Cp, c = e - w * Cp;
        float av = 0.f, sv = 0.f;
        if (c < C) {
            float conv = 0.f, S = 0.f;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const int ww = w + k - 5;
                if (ww >= 0 && ww < W) {
                    const float wk = q.w1[c * 11 + k];
                    conv = fmaf(wk, colsum_s[ww * C + c] * invH, conv);
                    S += wk;
                }
            }
            const float m = q.bn_m[c];
            av = (conv + q.b1[c]) * m + q.bn_a[c]; sv = S * m;
        }
        As[e] = av; Sms[e] = sv;
    }
    __syncthreads();
    // ---- masks of this block's rows, a thread owns LS_R vertically consecutive pixels of one column ---------------------------
    const int g = t / W, w = t - g * W;
    if (g >= groups) return;
    const int r0 = h0 + g * LS_R;                        // first row of this thread's strip
    if (r0 >= H) return;
    uint32_t valid = 0;                                  // bit j: row r0 - 5 + j lies inside the image
#pragma unroll
    for (int j = 0; j < LS_R + 10; ++j) valid |= (uint32_t)(r0 - 5 + j >= 0 && r0 - 5 + j < H) << j;
    float logit[LS_R][9];
#pragma unroll
    for (int r = 0; r < LS_R; ++r)
#pragma unroll
        for (int j = 0; j < 9; ++j) logit[r][j] = q.b3[j];
    const float4* A4 = reinterpret_cast<const float4*>(As + w * Cp);
    const float4* S4 = reinterpret_cast<const float4*>(Sms + w * Cp);
    const float4* w24 = reinterpret_cast<const float4*>(sw2);
    const float4* w34 = reinterpret_cast<const float4*>(sw3);
#pragma unroll 1
    for (int c4 = 0; c4 < (Cp >> 2); ++c4) {
        const float4 av = A4[c4], sv = S4[c4];
        const float aa[4] = {av.x, av.y, av.z, av.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const int c = 4 * c4 + j4;
            const float a = aa[j4], s = ss[j4];
            const float4* rm4 = reinterpret_cast<const float4*>(rm + c * P + g * LS_R);
            float tv[16];
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) { const float4 v4 = rm4[qq]; tv[4 * qq] = v4.x; tv[4 * qq + 1] = v4.y; tv[4 * qq + 2] = v4.z; tv[4 * qq + 3] = v4.w; }
#pragma unroll
            for (int j = 0; j < LS_R + 10; ++j) tv[j] = ((valid >> j) & 1u) ? fmaxf(fmaf(tv[j], s, a), 0.f) : 0.f;
            const float4 u0 = w24[3 * c], u1 = w24[3 * c + 1], u2 = w24[3 * c + 2];
            const float uk[11] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w, u2.x, u2.y, u2.z};
            const float4 q0 = w34[3 * c], q1 = w34[3 * c + 1], q2 = w34[3 * c + 2];
#pragma unroll
            for (int r = 0; r < LS_R; ++r) {
                float v = u2.w;       // bias of the 11x1 convolution (0 for a padding channel, whose weights are 0 as well)
#pragma unroll
                for (int k = 0; k < 11; ++k) v = fmaf(uk[k], tv[r + k], v);
                logit[r][0] = fmaf(q0.x, v, logit[r][0]); logit[r][1] = fmaf(q0.y, v, logit[r][1]); logit[r][2] = fmaf(q0.z, v, logit[r][2]);
                logit[r][3] = fmaf(q0.w, v, logit[r][3]); logit[r][4] = fmaf(q1.x, v, logit[r][4]); logit[r][5] = fmaf(q1.y, v, logit[r][5]);
                logit[r][6] = fmaf(q1.z, v, logit[r][6]); logit[r][7] = fmaf(q1.w, v, logit[r][7]); logit[r][8] = fmaf(q2.x, v, logit[r][8]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < LS_R; ++r) {
        if (r0 + r >= H) break;
        const size_t o = ((size_t)b * H * W + (size_t)(r0 + r) * W + w) * 9;
#pragma unroll
        for (int j = 0; j < 9; ++j) store_mixed<T>(q.mask, o + j, p.mask_f32, sigmoid_mask(logit[r][j]));
    }
}

// ------------------------------------------------------------------------------ SE
// Channel means from per-tile sums, by all 256 threads of a block and in a fixed order: K tiles are summed side by side
// (thread = (tile residue, channel), coalesced), then the K partial sums of a channel are added in order.
__device__ __forceinline__ int se_parallel_tiles(int tiles, int C) { return max(1, min(tiles, 256 / max(C, 1))); }
__device__ __forceinline__ void se_partial_sums(const float* __restrict__ gap_b, int tiles, int C, float* part, int tid) {
    const int K = se_parallel_tiles(tiles, C);
    for (int idx = tid; idx < K * C; idx += 256) {
        const int k0 = idx / C, c = idx - k0 * C;
        float s = 0.f;
        for (int k = k0; k < tiles; k += K) s += gap_b[(size_t)k * C + c];
        part[idx] = s;
    }
}
__device__ __forceinline__ float se_mean_of(const float* part, int tiles, int C, int c, float inv_count) {
    const int K = se_parallel_tiles(tiles, C);
    float s = 0.f;
    for (int k0 = 0; k0 < K; ++k0) s += part[k0 * C + c];
    return s * inv_count;
}

// 256 threads per image
__global__ void __launch_bounds__(256)
se_excite_kernel(const float* __restrict__ gap_partial, int tiles, float inv_count,
                 const float* __restrict__ w1, const float* __restrict__ b1,
                 const float* __restrict__ w2, const float* __restrict__ b2,
                 float* __restrict__ att, int C, int Hd) {
    extern __shared__ float sm[];
    float* mean = sm;                    // [C]
    float* hid = sm + C;                 // [Hd]
    float* part = hid + Hd;              // [max(256, C)]
    int b = blockIdx.x, t = threadIdx.x;
    grid_dependency_wait();              // the channel sums come from the kernel before
    grid_dependents_go();
    se_partial_sums(gap_partial + (size_t)b * tiles * C, tiles, C, part, t);
    __syncthreads();
    for (int c = t; c < C; c += 256) mean[c] = se_mean_of(part, tiles, C, c, inv_count);
    __syncthreads();
    for (int h = t; h < Hd; h += 256) {
        float s = b1[h];
        for (int c = 0; c < C; ++c) s = fmaf(w1[(size_t)h * C + c], mean[c], s);
        hid[h] = fmaxf(s, 0.f);
    }
    __syncthreads();
    for (int c = t; c < C; c += 256) {
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

// V consecutive channels as floats (V = 1, or V = 2 for 16-bit types: one 32-bit access)
template <typename T, int V> struct MergeIO {
    static __device__ __forceinline__ void ld(const T* p, float (&o)[V]) { o[0] = to_f<T>(*p); }
    static __device__ __forceinline__ void st(T* p, const float (&v)[V]) { *p = from_f<T>(v[0]); }
};
template <> struct MergeIO<__half, 2> {
    static __device__ __forceinline__ void ld(const __half* p, float (&o)[2]) { float2 f = __half22float2(*reinterpret_cast<const __half2*>(p)); o[0] = f.x; o[1] = f.y; }
    static __device__ __forceinline__ void st(__half* p, const float (&v)[2]) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(v[0], v[1]); }
};
template <> struct MergeIO<__nv_bfloat16, 2> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&o)[2]) { float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); o[0] = f.x; o[1] = f.y; }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[2]) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]); }
};

// blockDim = 256 = (pixel lanes) x (channel groups rounded up to a power of two): a thread keeps its V channels (so its
// branch, its attention scalars and its source tensor are fixed per image) and walks over pixels; consecutive threads
// touch consecutive channels of the same pixel, i.e. consecutive addresses of x, out and the branch tensor.
template <typename T, int V>
__global__ void __launch_bounds__(256)
merge_kernel(const T* __restrict__ x, T* __restrict__ out, MergeParams p, int Cp, int pix_per_block, int out_ld) {
    const int cl0 = threadIdx.x % Cp, pl = threadIdx.x / Cp, PL = 256 / Cp;
    const int b = blockIdx.y;
    const int HW = p.H * p.W;
    const int pix0 = blockIdx.x * pix_per_block, pix1 = min(HW, pix0 + pix_per_block);
    for (int c = cl0 * V; c < p.C; c += Cp * V) {
        int i = 0, cl = c;
        if (cl >= p.c[0]) { cl -= p.c[0]; i = 1; if (cl >= p.c[1]) { cl -= p.c[1]; i = 2; } }
        // (selected by value: indexing the parameter arrays with a run-time i would move them to local memory)
        const int ci = i == 0 ? p.c[0] : (i == 1 ? p.c[1] : p.c[2]), hi = i == 0 ? p.h[0] : (i == 1 ? p.h[1] : p.h[2]);
        const int wi = i == 0 ? p.w[0] : (i == 1 ? p.w[1] : p.w[2]);
        const T* yi = reinterpret_cast<const T*>(i == 0 ? p.y[0] : (i == 1 ? p.y[1] : p.y[2])) + (size_t)b * hi * wi * ci + cl;
        const float* ai = i == 0 ? p.att[0] : (i == 1 ? p.att[1] : p.att[2]);
        float a[V];
#pragma unroll
        for (int v = 0; v < V; ++v) a[v] = ai[(size_t)b * ci + cl + v];
        const bool same = (hi == p.H && wi == p.W);
        const float sy = i == 0 ? p.sy[0] : (i == 1 ? p.sy[1] : p.sy[2]), sx = i == 0 ? p.sx[0] : (i == 1 ? p.sx[1] : p.sx[2]);
        for (int pix = pix0 + pl; pix < pix1; pix += PL) {
            const int yh = pix / p.W, xw = pix - yh * p.W;
            float val[V];
            if (same) {
                MergeIO<T, V>::ld(yi + (size_t)pix * ci, val);
            } else {
                int y0, y1, x0, x1; float ly, lx;
                src_index(yh, sy, hi, y0, y1, ly);
                src_index(xw, sx, wi, x0, x1, lx);
                float v00[V], v01[V], v10[V], v11[V];
                MergeIO<T, V>::ld(yi + ((size_t)y0 * wi + x0) * ci, v00); MergeIO<T, V>::ld(yi + ((size_t)y0 * wi + x1) * ci, v01);
                MergeIO<T, V>::ld(yi + ((size_t)y1 * wi + x0) * ci, v10); MergeIO<T, V>::ld(yi + ((size_t)y1 * wi + x1) * ci, v11);
#pragma unroll
                for (int v = 0; v < V; ++v)
                    val[v] = (1.f - ly) * ((1.f - lx) * v00[v] + lx * v01[v]) + ly * ((1.f - lx) * v10[v] + lx * v11[v]);
            }
            const size_t e = ((size_t)b * HW + pix) * p.C + c;
            float xin[V], o[V];
            MergeIO<T, V>::ld(x + e, xin);
#pragma unroll
            for (int v = 0; v < V; ++v) o[v] = fmaf(val[v], a[v], xin[v]);
            MergeIO<T, V>::st(out + ((size_t)b * HW + pix) * out_ld + c, o);
        }
    }
}

// The same tail for 16-bit tensors with C % 8 == 0: a thread owns one 16-byte vector (8 channels of one pixel) of x and
// out, so both are read and written fully coalesced; the branch values are gathered per channel (2-byte loads that hit
// L1: neighbouring pixels share their sources). Optionally the squeeze-excite MLP of the three branches is evaluated at
// the head of every block (a few hundred FMAs) from the channel sums the DSC kernels left behind, in the same order of
// operations as se_excite_kernel, so the attention never makes a trip through memory or a launch of its own.
struct MergeSe {
    const float* gap[3]; const float* w1[3]; const float* b1[3]; const float* w2[3]; const float* b2[3];
    int tiles[3], hidden[3];
    float inv[3];
};

// Attention of the three branches of one image into att_s[C] (channel order of the concatenation): either copied from
// memory, or the squeeze-excite MLP evaluated here from the channel sums, with the arithmetic of se_excite_kernel.
// scratch: mean[C] | hid[hidden0 + hidden1 + hidden2] | part[3][256]; every branch width <= 256.
__device__ __forceinline__ void merge_attention(const MergeParams& p, const MergeSe& se, int use_se, int b, float* att_s, float* scratch, int tid) {
    const int c0 = p.c[0], c1 = p.c[1], c2 = p.c[2];
    if (!use_se) {
        for (int c = tid; c < c0; c += 256) att_s[c] = p.att[0][(size_t)b * c0 + c];
        for (int c = tid; c < c1; c += 256) att_s[c0 + c] = p.att[1][(size_t)b * c1 + c];
        for (int c = tid; c < c2; c += 256) att_s[c0 + c1 + c] = p.att[2][(size_t)b * c2 + c];
        __syncthreads();
        return;
    }
    float* mean = scratch;
    float* hid = mean + p.C;
    float* part = hid + se.hidden[0] + se.hidden[1] + se.hidden[2];
    se_partial_sums(se.gap[0] + (size_t)b * se.tiles[0] * c0, se.tiles[0], c0, part, tid);
    se_partial_sums(se.gap[1] + (size_t)b * se.tiles[1] * c1, se.tiles[1], c1, part + 256, tid);
    se_partial_sums(se.gap[2] + (size_t)b * se.tiles[2] * c2, se.tiles[2], c2, part + 512, tid);
    __syncthreads();
    for (int c = tid; c < p.C; c += 256) {
        if (c < c0) mean[c] = se_mean_of(part, se.tiles[0], c0, c, se.inv[0]);
        else if (c < c0 + c1) mean[c] = se_mean_of(part + 256, se.tiles[1], c1, c - c0, se.inv[1]);
        else mean[c] = se_mean_of(part + 512, se.tiles[2], c2, c - c0 - c1, se.inv[2]);
    }
    __syncthreads();
    const int h0 = se.hidden[0], h1 = se.hidden[1], h2 = se.hidden[2];
    for (int h = tid; h < h0 + h1 + h2; h += 256) {
        const int i = h < h0 ? 0 : (h < h0 + h1 ? 1 : 2);
        const int hl = i == 0 ? h : (i == 1 ? h - h0 : h - h0 - h1), ci = i == 0 ? c0 : (i == 1 ? c1 : c2), cb = i == 0 ? 0 : (i == 1 ? c0 : c0 + c1);
        const float* w1 = i == 0 ? se.w1[0] : (i == 1 ? se.w1[1] : se.w1[2]);
        const float* b1 = i == 0 ? se.b1[0] : (i == 1 ? se.b1[1] : se.b1[2]);
        float s = b1[hl];
        for (int c = 0; c < ci; ++c) s = fmaf(w1[(size_t)hl * ci + c], mean[cb + c], s);
        hid[h] = fmaxf(s, 0.f);
    }
    __syncthreads();
    for (int c = tid; c < p.C; c += 256) {
        const int i = c < c0 ? 0 : (c < c0 + c1 ? 1 : 2);
        const int cl = i == 0 ? c : (i == 1 ? c - c0 : c - c0 - c1), Hd = i == 0 ? h0 : (i == 1 ? h1 : h2), hb = i == 0 ? 0 : (i == 1 ? h0 : h0 + h1);
        const float* w2 = i == 0 ? se.w2[0] : (i == 1 ? se.w2[1] : se.w2[2]);
        const float* b2 = i == 0 ? se.b2[0] : (i == 1 ? se.b2[1] : se.b2[2]);
        float s = b2[cl];
        for (int h = 0; h < Hd; ++h) s = fmaf(w2[(size_t)cl * Hd + h], hid[hb + h], s);
        att_s[c] = sigmoidf_(s);
    }
    __syncthreads();
}

template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
template <typename T> __device__ __forceinline__ uint32_t pack2f(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2f<__half>(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
template <> __device__ __forceinline__ uint32_t pack2f<__nv_bfloat16>(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }

struct BranchTap { int o00, o01, o10, o11; float ly, lx; };

template <typename T>
__global__ void __launch_bounds__(256)
merge_vec8_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, MergeParams p, MergeSe se, int use_se, int G, int PL,
                  int pix_per_block, int out_ld8) {
    extern __shared__ float sm_merge[];
    float* att_s = sm_merge;             // [C] attention of this image, channel order of the concatenation
    const int b = blockIdx.y, tid = threadIdx.x;
    merge_attention(p, se, use_se, b, att_s, att_s + p.C, tid);
    const int grp = tid % G, pl = tid / G;
    if (pl >= PL) return;
    const int HW = p.H * p.W;
    // the 8 channels of this thread: branch, channel inside the branch, attention
    int bi[8], cl[8]; float at[8];
    int uses = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int c = grp * 8 + j, i = 0;
        at[j] = att_s[c];
        if (c >= p.c[0]) { c -= p.c[0]; i = 1; if (c >= p.c[1]) { c -= p.c[1]; i = 2; } }
        bi[j] = i; cl[j] = c; uses |= 1 << i;
    }
    const T* yb[3]; int cc[3]; bool same[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        cc[i] = p.c[i];
        yb[i] = reinterpret_cast<const T*>(p.y[i]) + (size_t)b * p.h[i] * p.w[i] * cc[i];
        same[i] = p.h[i] == p.H && p.w[i] == p.W;
    }
    const int pix0 = blockIdx.x * pix_per_block, pix1 = min(HW, pix0 + pix_per_block);
    for (int pix = pix0 + pl; pix < pix1; pix += PL) {
        const int yh = pix / p.W, xw = pix - yh * p.W;
        const uint4 xv = x[((size_t)b * HW + pix) * G + grp];
        BranchTap bt[3];
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            if (!((uses >> i) & 1)) continue;
            if (same[i]) { bt[i].o00 = bt[i].o01 = bt[i].o10 = bt[i].o11 = pix * cc[i]; bt[i].ly = bt[i].lx = 0.f; continue; }
            int y0, y1, x0, x1;
            src_index(yh, p.sy[i], p.h[i], y0, y1, bt[i].ly);
            src_index(xw, p.sx[i], p.w[i], x0, x1, bt[i].lx);
            bt[i].o00 = (y0 * p.w[i] + x0) * cc[i]; bt[i].o01 = (y0 * p.w[i] + x1) * cc[i];
            bt[i].o10 = (y1 * p.w[i] + x0) * cc[i]; bt[i].o11 = (y1 * p.w[i] + x1) * cc[i];
        }
        float val[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // (values are selected, never references: the per-branch state has to stay in registers)
            const int i = bi[j];
            const int o00 = i == 0 ? bt[0].o00 : (i == 1 ? bt[1].o00 : bt[2].o00), o01 = i == 0 ? bt[0].o01 : (i == 1 ? bt[1].o01 : bt[2].o01);
            const int o10 = i == 0 ? bt[0].o10 : (i == 1 ? bt[1].o10 : bt[2].o10), o11 = i == 0 ? bt[0].o11 : (i == 1 ? bt[1].o11 : bt[2].o11);
            const float ly = i == 0 ? bt[0].ly : (i == 1 ? bt[1].ly : bt[2].ly), lx = i == 0 ? bt[0].lx : (i == 1 ? bt[1].lx : bt[2].lx);
            const T* yi = (i == 0 ? yb[0] : (i == 1 ? yb[1] : yb[2])) + cl[j];
            const bool sm_ = i == 0 ? same[0] : (i == 1 ? same[1] : same[2]);
            if (sm_) {
                val[j] = to_f<T>(yi[o00]);
            } else {
                const float v00 = to_f<T>(yi[o00]), v01 = to_f<T>(yi[o01]), v10 = to_f<T>(yi[o10]), v11 = to_f<T>(yi[o11]);
                val[j] = (1.f - ly) * ((1.f - lx) * v00 + lx * v01) + ly * ((1.f - lx) * v10 + lx * v11);
            }
        }
        const float2 x0 = unpack2<T>(xv.x), x1 = unpack2<T>(xv.y), x2 = unpack2<T>(xv.z), x3 = unpack2<T>(xv.w);
        uint4 o;
        o.x = pack2f<T>(fmaf(val[0], at[0], x0.x), fmaf(val[1], at[1], x0.y));
        o.y = pack2f<T>(fmaf(val[2], at[2], x1.x), fmaf(val[3], at[3], x1.y));
        o.z = pack2f<T>(fmaf(val[4], at[4], x2.x), fmaf(val[5], at[5], x2.y));
        o.w = pack2f<T>(fmaf(val[6], at[6], x3.x), fmaf(val[7], at[7], x3.y));
        out[((size_t)b * HW + pix) * out_ld8 + grp] = o;
    }
}

// The tail for 16-bit tensors with the branch rows staged in shared memory, in two phases. A block owns R consecutive
// output rows of one image. The source rows those outputs interpolate from are, for every branch, ONE contiguous run of
// the NHWC branch tensor, copied to shared memory with 16-byte accesses (the run keeps its offset from a 16-byte
// boundary, the ragged ends go as 2-byte elements).
//   phase 0  the x rows are copied into an output tile in shared memory (coalesced)
//   phase 1  one work item per (branch, pixel): the interpolation geometry is computed once and reused for all channels
//            of the branch; tile = tile + att * upsample(y), formed in fp32
//   phase 2  the tile leaves coalesced (out may be a channel slice of a wider tensor).
// PAIRS: every branch width is even, so channels are handled two at a time with 4-byte accesses.
constexpr int MERGE_CHUNK = 12;     // channels per work item of phase 1 (even)
struct MergeStage { int off[3]; int cap_rows[3]; int tile_off; };     // byte offsets of the branch regions and the tile

__device__ __forceinline__ void cp_async_bytes16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_bytes4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_everything() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// (asynchronous: the caller waits with cp_async_wait_everything() and a barrier)
__device__ __forceinline__ void copy_run_to_smem(unsigned char* dst, const unsigned char* src, int nbytes, int tid) {
    // dst and src have the same offset from a 16-byte boundary; nbytes is even
    const int head = min(nbytes, static_cast<int>((16 - (reinterpret_cast<uintptr_t>(src) & 15)) & 15));
    const int body = (nbytes - head) >> 4, tail = nbytes - head - (body << 4);
    const uint4* s4 = reinterpret_cast<const uint4*>(src + head);
    uint4* d4 = reinterpret_cast<uint4*>(dst + head);
    for (int i = tid; i < body; i += 256) cp_async_bytes16(d4 + i, s4 + i);
    if (tid < (head >> 1)) reinterpret_cast<uint16_t*>(dst)[tid] = reinterpret_cast<const uint16_t*>(src)[tid];
    else if (tid >= 32 && tid - 32 < (tail >> 1))
        reinterpret_cast<uint16_t*>(dst + head + (body << 4))[tid - 32] = reinterpret_cast<const uint16_t*>(src + head + (body << 4))[tid - 32];
}

// One branch of phase 1 (i is a compile-time constant at every call site, so nothing is indexed at run time).
template <typename T, bool PAIRS>
__device__ __forceinline__ void merge_branch(const T* __restrict__ ysrc, T* __restrict__ tile, const float* __restrict__ att,
                                             int c, int cbase, int hi, int wi, float sy, float sx, int lo, bool same,
                                             int pitch, int W, int row0, int npx, int tid) {
    // work item = (pixel, chunk of MERGE_CHUNK channels): consecutive lanes take consecutive pixels
    const int nchunk = (c + MERGE_CHUNK - 1) / MERGE_CHUNK;
    for (int item = tid; item < npx * nchunk; item += 256) {
        const int chunk = item / npx, q = item - chunk * npx;
        const int ch_lo = chunk * MERGE_CHUNK, ch_hi = min(c, ch_lo + MERGE_CHUNK);
        const int yh = row0 + q / W, xw = q % W;
        int o00, o01, o10, o11; float ly = 0.f, lx = 0.f;
        if (same) { o00 = o01 = o10 = o11 = ((yh - lo) * wi + xw) * c; }
        else {
            int y0, y1, x0, x1;
            src_index(yh, sy, hi, y0, y1, ly);
            src_index(xw, sx, wi, x0, x1, lx);
            y0 -= lo; y1 -= lo;
            o00 = (y0 * wi + x0) * c; o01 = (y0 * wi + x1) * c; o10 = (y1 * wi + x0) * c; o11 = (y1 * wi + x1) * c;
        }
        T* tp = tile + (size_t)q * pitch + cbase;      // holds x on entry, out on exit
        if (PAIRS) {
            for (int ch = ch_lo; ch < ch_hi; ch += 2) {
                const float2 xin = unpack2<T>(*reinterpret_cast<const uint32_t*>(tp + ch));
                float2 v;
                if (same) v = unpack2<T>(*reinterpret_cast<const uint32_t*>(ysrc + o00 + ch));
                else {
                    const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(ysrc + o00 + ch)), b = unpack2<T>(*reinterpret_cast<const uint32_t*>(ysrc + o01 + ch));
                    const float2 d = unpack2<T>(*reinterpret_cast<const uint32_t*>(ysrc + o10 + ch)), e = unpack2<T>(*reinterpret_cast<const uint32_t*>(ysrc + o11 + ch));
                    v.x = (1.f - ly) * ((1.f - lx) * a.x + lx * b.x) + ly * ((1.f - lx) * d.x + lx * e.x);
                    v.y = (1.f - ly) * ((1.f - lx) * a.y + lx * b.y) + ly * ((1.f - lx) * d.y + lx * e.y);
                }
                *reinterpret_cast<uint32_t*>(tp + ch) = pack2f<T>(fmaf(v.x, att[ch], xin.x), fmaf(v.y, att[ch + 1], xin.y));
            }
        } else {
            for (int ch = ch_lo; ch < ch_hi; ++ch) {
                const float xin = to_f<T>(tp[ch]);
                float v;
                if (same) v = to_f<T>(ysrc[o00 + ch]);
                else v = (1.f - ly) * ((1.f - lx) * to_f<T>(ysrc[o00 + ch]) + lx * to_f<T>(ysrc[o01 + ch])) +
                         ly * ((1.f - lx) * to_f<T>(ysrc[o10 + ch]) + lx * to_f<T>(ysrc[o11 + ch]));
                tp[ch] = from_f<T>(fmaf(v, att[ch], xin));
            }
        }
    }
}

// The tail for 16-bit tensors without shared memory: a thread OWNS a group of four consecutive channels of ONE branch (so its
// source tensor, its attention scalars and, for a pooled branch, the horizontal interpolation of its column are fixed) and one
// column x of a strip of the image, and walks down the rows of the block. Groups never straddle a branch: branch i has
// ceil(c_i / 4) groups, and when c_i is no multiple of four its last group is the LAST four channels of the branch (it
// overlaps its neighbour and stores only the channels that neighbour does not cover), so every thread runs the same
// vector code. Consecutive threads hold consecutive groups of the same pixel and then the next pixel: x and out are read and
// written as (nearly) contiguous 8-byte pieces; the branch values come through L1 / L2 (a pooled branch is read four or
// sixteen times, by neighbouring threads and rows). Attention values are read from memory (att[i][b][c]).
// ALIGN: guaranteed alignment in bytes of every group's address in x, out and the branch tensors (8, 4 or 2).
template <typename T, int ALIGN>
__global__ void __launch_bounds__(256)
merge_col_kernel(const T* __restrict__ x, T* __restrict__ out, MergeParams p, int G, int PL, int R, int out_ld) {
    const int tid = threadIdx.x;
    grid_dependency_wait();              // branch tensors and attention values come from the kernels before
    grid_dependents_go();
    if (tid >= G * PL) return;
    const int g = tid % G, pl = tid / G, b = blockIdx.z;
    const int xw = blockIdx.x * PL + pl;
    if (xw >= p.W) return;
    const int row0 = blockIdx.y * R, row1 = min(p.H, row0 + R);
    const int HW = p.H * p.W;
    const int c0 = p.c[0], c1 = p.c[1], g0 = (c0 + 3) >> 2, g1 = (c1 + 3) >> 2;
    const int i = g < g0 ? 0 : (g < g0 + g1 ? 1 : 2);
    const int ci = i == 0 ? c0 : (i == 1 ? c1 : p.c[2]), hi = i == 0 ? p.h[0] : (i == 1 ? p.h[1] : p.h[2]);
    const int wi = i == 0 ? p.w[0] : (i == 1 ? p.w[1] : p.w[2]);
    const int lg = g - (i == 0 ? 0 : (i == 1 ? g0 : g0 + g1));
    const int lc = min(4 * lg, ci - 4), skip = 4 * lg - lc;             // first channel of the group inside the branch; channels to leave alone
    const int ch0 = (i == 0 ? 0 : (i == 1 ? c0 : c0 + c1)) + lc;
    const float sy = i == 0 ? p.sy[0] : (i == 1 ? p.sy[1] : p.sy[2]), sx = i == 0 ? p.sx[0] : (i == 1 ? p.sx[1] : p.sx[2]);
    const unsigned char* yb = reinterpret_cast<const unsigned char*>(reinterpret_cast<const T*>(i == 0 ? p.y[0] : (i == 1 ? p.y[1] : p.y[2])) + (size_t)b * hi * wi * ci + lc);
    const float* ai = (i == 0 ? p.att[0] : (i == 1 ? p.att[1] : p.att[2])) + (size_t)b * ci + lc;
    const float a0 = ai[0], a1 = ai[1], a2 = ai[2], a3 = ai[3];
    const bool same = hi == p.H && wi == p.W;
    int x0 = xw, x1 = xw; float lx = 0.f;
    if (!same) src_index(xw, sx, wi, x0, x1, lx);
    const float hx = 1.f - lx;
    const unsigned char* xp = reinterpret_cast<const unsigned char*>(x + ((size_t)b * HW + (size_t)row0 * p.W + xw) * p.C + ch0);
    T* op = out + ((size_t)b * HW + (size_t)row0 * p.W + xw) * out_ld + ch0;
    const size_t xstep = 2 * (size_t)p.W * p.C, ostep = (size_t)p.W * out_ld;
    // stores one row's group (the channels of an overlapping last group that the neighbour covers are left alone)
    auto put = [&](T* o, uint32_t lo, uint32_t hi2) {
        if (skip == 0) {
            if (ALIGN == 8) *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi2);
            else if (ALIGN == 4) { reinterpret_cast<uint32_t*>(o)[0] = lo; reinterpret_cast<uint32_t*>(o)[1] = hi2; }
            else { uint16_t* o16 = reinterpret_cast<uint16_t*>(o); o16[0] = (uint16_t)lo; o16[1] = (uint16_t)(lo >> 16); o16[2] = (uint16_t)hi2; o16[3] = (uint16_t)(hi2 >> 16); }
        } else if (skip == 2 && ALIGN >= 4) {
            reinterpret_cast<uint32_t*>(o)[1] = hi2;
        } else {
            uint16_t* o16 = reinterpret_cast<uint16_t*>(o);
            if (skip <= 1) o16[1] = (uint16_t)(lo >> 16);
            if (skip <= 2) o16[2] = (uint16_t)hi2;
            o16[3] = (uint16_t)(hi2 >> 16);
        }
    };
    // Two rows per trip, all loads of both rows issued before the first use (the loop is bound by load latency, not by bandwidth).
    // A warp holds groups of the full-resolution branch and of the pooled ones side by side: ONE loop for both kinds, so that the
    // loads of either kind are in flight together (two loops would run one after the other with half the lanes masked).
    const unsigned char* yp = yb + 2 * ((size_t)row0 * wi + xw) * ci;          // full-resolution branch: this pixel in row row0
    const size_t ystep = 2 * (size_t)wi * ci;
    const unsigned char* c0p = yb + 2 * x0 * ci;
    const unsigned char* c1p = yb + 2 * x1 * ci;
    // one row of a pooled branch: the four corner groups, the blend
    auto blend_row = [&](uint2 xin, uint2 q00, uint2 q01, uint2 q10, uint2 q11, float ly, T* o) {
        const float hy = 1.f - ly;
        const float2 xa = unpack2<T>(xin.x), xb = unpack2<T>(xin.y);
        const float2 a00 = unpack2<T>(q00.x), b00 = unpack2<T>(q00.y), a01 = unpack2<T>(q01.x), b01 = unpack2<T>(q01.y);
        const float2 a10 = unpack2<T>(q10.x), b10 = unpack2<T>(q10.y), a11 = unpack2<T>(q11.x), b11 = unpack2<T>(q11.y);
        const float v0 = hy * (hx * a00.x + lx * a01.x) + ly * (hx * a10.x + lx * a11.x);
        const float v1 = hy * (hx * a00.y + lx * a01.y) + ly * (hx * a10.y + lx * a11.y);
        const float v2 = hy * (hx * b00.x + lx * b01.x) + ly * (hx * b10.x + lx * b11.x);
        const float v3 = hy * (hx * b00.y + lx * b01.y) + ly * (hx * b10.y + lx * b11.y);
        put(o, pack2f<T>(fmaf(v0, a0, xa.x), fmaf(v1, a1, xa.y)), pack2f<T>(fmaf(v2, a2, xb.x), fmaf(v3, a3, xb.y)));
    };
    auto same_row = [&](uint2 xin, uint2 v, T* o) {
        const float2 xa = unpack2<T>(xin.x), xb = unpack2<T>(xin.y), va = unpack2<T>(v.x), vb = unpack2<T>(v.y);
        put(o, pack2f<T>(fmaf(va.x, a0, xa.x), fmaf(va.y, a1, xa.y)), pack2f<T>(fmaf(vb.x, a2, xb.x), fmaf(vb.y, a3, xb.y)));
    };
    int yh = row0;
    for (; yh + 1 < row1; yh += 2, xp += 2 * xstep, op += 2 * ostep, yp += 2 * ystep) {
        const uint2 xi0 = ldg8<ALIGN>(xp), xi1 = ldg8<ALIGN>(xp + xstep);
        uint2 p00, p01, p10, p11, r00, r01, r10, r11;
        float lya = 0.f, lyb = 0.f;
        if (same) {
            p00 = ldg8<ALIGN>(yp); r00 = ldg8<ALIGN>(yp + ystep);
            p01 = p10 = p11 = r01 = r10 = r11 = make_uint2(0u, 0u);
        } else {
            int ya0, ya1, yb0, yb1;
            src_index(yh, sy, hi, ya0, ya1, lya);
            src_index(yh + 1, sy, hi, yb0, yb1, lyb);
            p00 = ldg8<ALIGN>(c0p + ya0 * ystep); p01 = ldg8<ALIGN>(c1p + ya0 * ystep); p10 = ldg8<ALIGN>(c0p + ya1 * ystep); p11 = ldg8<ALIGN>(c1p + ya1 * ystep);
            r00 = ldg8<ALIGN>(c0p + yb0 * ystep); r01 = ldg8<ALIGN>(c1p + yb0 * ystep); r10 = ldg8<ALIGN>(c0p + yb1 * ystep); r11 = ldg8<ALIGN>(c1p + yb1 * ystep);
        }
        if (same) { same_row(xi0, p00, op); same_row(xi1, r00, op + ostep); }
        else { blend_row(xi0, p00, p01, p10, p11, lya, op); blend_row(xi1, r00, r01, r10, r11, lyb, op + ostep); }
    }
    if (yh < row1) {
        const uint2 xi0 = ldg8<ALIGN>(xp);
        if (same) same_row(xi0, ldg8<ALIGN>(yp), op);
        else {
            int ya0, ya1; float lya;
            src_index(yh, sy, hi, ya0, ya1, lya);
            const uint2 p00 = ldg8<ALIGN>(c0p + ya0 * ystep), p01 = ldg8<ALIGN>(c1p + ya0 * ystep), p10 = ldg8<ALIGN>(c0p + ya1 * ystep), p11 = ldg8<ALIGN>(c1p + ya1 * ystep);
            blend_row(xi0, p00, p01, p10, p11, lya, op);
        }
    }
}

template <typename T, bool PAIRS>
__global__ void __launch_bounds__(256)
merge_tile_kernel(const T* __restrict__ x, uint4* __restrict__ out, MergeParams p, MergeSe se, MergeStage stg, int use_se, int R, int out_ld8,
                  int se_floats) {
    extern __shared__ __align__(16) unsigned char sm_rows[];
    float* att_s = reinterpret_cast<float*>(sm_rows);      // [C], then the scratch of merge_attention
    unsigned char* stage = sm_rows + se_floats * 4;
    T* tile = reinterpret_cast<T*>(stage + stg.tile_off);
    const int b = blockIdx.y, tid = threadIdx.x;
    const int row0 = blockIdx.x * R, row1 = min(p.H, row0 + R);
    const int HW = p.H * p.W, npx = (row1 - row0) * p.W;

    // x rows -> the output tile. A pixel of the tile is C/2 + 1 words long: phase 1 runs one thread per pixel, and an odd
    // pitch keeps its 32 lanes on 32 different banks (a pitch of C/2 words would be a 16- or 32-way conflict).
    const int Cw = p.C >> 1, pitch_w = Cw + 1, pitch = 2 * pitch_w;
    const bool pow2 = (Cw & (Cw - 1)) == 0;
    const int sh = 31 - __clz(Cw);
    {
        const uint32_t* xs = reinterpret_cast<const uint32_t*>(x + ((size_t)b * HW + (size_t)row0 * p.W) * p.C);
        uint32_t* tw = reinterpret_cast<uint32_t*>(tile);
        for (int w = tid; w < npx * Cw; w += 256) {
            const int q = pow2 ? (w >> sh) : (w / Cw);
            cp_async_bytes4(tw + q * pitch_w + (w - q * Cw), xs + w);
        }
    }
    // source rows of every branch -> shared memory
    const T* src[3]; int lo[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int hi_ = p.h[i], wi = p.w[i], ci = p.c[i];
        const bool same = hi_ == p.H && wi == p.W;
        int first, last;
        if (same) { first = row0; last = row1 - 1; }
        else {
            int a0, a1, b0, b1; float l;
            src_index(row0, p.sy[i], hi_, a0, a1, l);
            src_index(row1 - 1, p.sy[i], hi_, b0, b1, l);
            first = a0; last = b1;
        }
        const T* g = reinterpret_cast<const T*>(p.y[i]) + (size_t)b * hi_ * wi * ci;
        if (last - first + 1 <= stg.cap_rows[i]) {
            const unsigned char* run = reinterpret_cast<const unsigned char*>(g + (size_t)first * wi * ci);
            unsigned char* dst = stage + stg.off[i] + (reinterpret_cast<uintptr_t>(run) & 15);
            copy_run_to_smem(dst, run, (last - first + 1) * wi * ci * 2, tid);
            src[i] = reinterpret_cast<const T*>(dst); lo[i] = first;
        } else {                                            // (never with the capacities the host computes)
            src[i] = g; lo[i] = 0;
        }
    }
    merge_attention(p, se, use_se, b, att_s, att_s + p.C, tid);      // (overlaps the copies in flight)
    cp_async_wait_everything();
    __syncthreads();
    int cbase;

    cbase = 0;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        merge_branch<T, PAIRS>(src[i], tile, att_s + cbase, p.c[i], cbase, p.h[i], p.w[i], p.sy[i], p.sx[i], lo[i],
                               p.h[i] == p.H && p.w[i] == p.W, pitch, p.W, row0, npx, tid);
        cbase += p.c[i];
    }
    __syncthreads();
    const uint32_t* tr = reinterpret_cast<const uint32_t*>(tile);
    uint32_t* orow = reinterpret_cast<uint32_t*>(out + ((size_t)b * HW + (size_t)row0 * p.W) * out_ld8);
    const int out_w = out_ld8 * 4;                          // words per pixel of out
    for (int w = tid; w < npx * Cw; w += 256) {
        const int q = pow2 ? (w >> sh) : (w / Cw), k = w - q * Cw;
        orow[(size_t)q * out_w + k] = tr[q * pitch_w + k];
    }
}

// avg-pool (pool x pool, stride pool, floor), NHWC; one thread per output pixel and channel.
template <typename T>
__global__ void avg_pool_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int Ho, int Wo, int C, int pool, size_t n) {
    const float inv = 1.f / (float)(pool * pool);
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % C);
        size_t r = e / C;
        const int xo = (int)(r % Wo); r /= Wo;
        const int yo = (int)(r % Ho); const int b = (int)(r / Ho);
        const T* base = x + (((size_t)b * H + yo * pool) * W + xo * pool) * C + c;
        float s = 0.f;
        for (int dy = 0; dy < pool; ++dy)
            for (int dx = 0; dx < pool; ++dx) s += to_f<T>(base[((size_t)dy * W + dx) * C]);
        y[e] = from_f<T>(s * inv);
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
    size_t smem = sizeof(float) * (size_t)36 * C;
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

extern "C" int kad_lcsa_mask_from_partials_supported(int H, int W, int C) {
    if (H <= 0 || W <= 0 || C <= 0) return 0;
    const int nrows = (127 / W + 2) < H ? (127 / W + 2) : H;
    return C <= 256 && (size_t)(2 * nrows + 1) * 12 * ((C + 3) & ~3) * 4 <= 96 * 1024;
}

extern "C" int kad_lcsa_mask_from_partials(const float* rowpart, int n_col_tiles, const float* colpart, int n_row_groups,
                                           const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                                           const float* w2, const float* b2, const float* w3, const float* b3,
                                           float* scratch, float* rowsum, void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream) {
    KAD_CHECK_ARG(rowpart && colpart && w1 && b1 && bn_scale && bn_shift && w2 && b2 && w3 && b3 && scratch && rowsum && mask,
                  "kad_lcsa_mask_from_partials: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && C > 0 && B <= 65535 && n_col_tiles > 0 && n_row_groups > 0, "kad_lcsa_mask_from_partials: bad shape");
    if (!kad_lcsa_mask_from_partials_supported(H, W, C))
        return fail(KAD_ERR_UNSUPPORTED, "kad_lcsa_mask_from_partials: C = %d, W = %d exceed the shared-memory staging", C, W);
    cudaStream_t st = (cudaStream_t)stream;
    const int Cp = (C + 3) & ~3;          // scratch: A [B][W][Cp] then Sm [W][Cp]
    KAD_CHECK_ARG((uintptr_t)scratch % 16 == 0, "kad_lcsa_mask_from_partials: scratch must be 16-byte aligned");
    float* A = scratch;
    float* Sm = scratch + (size_t)B * W * Cp;
    launch_pdl(lcsa_prep_partials_kernel, dim3((W + PREP_COLS - 1) / PREP_COLS, B), 256, sizeof(float) * (size_t)(PREP_COLS + 10) * C, st,
               rowpart, n_col_tiles, colpart, n_row_groups, w1, b1, bn_scale, bn_shift, A, Sm, rowsum, H, W, C, Cp);
    return kad::lcsa_mask_from_prepared(rowsum, 0, A, Sm, w2, b2, w3, b3, mask, B, H, W, C, mask_f32, dtype, st);
}

// The second stage of the LCSA (11x1 depthwise, 1x1, sigmoid) from prepared first-stage operands: rows float32 [B][H][C] (row sums,
// or row means when rows_are_means), A [B][W][Cp], Sm [W][Cp]. One launch.
int kad::lcsa_mask_from_prepared(const float* rowsum, int rows_are_means, const float* A, const float* Sm,
                                 const float* w2, const float* b2, const float* w3, const float* b3,
                                 void* mask, int B, int H, int W, int C, int mask_f32, int dtype, cudaStream_t st) {
    const int Cp = (C + 3) & ~3;
    // float32 masks at a 16-byte aligned address leave through shared memory, as 16-byte stores in global order
    const int staged = mask_f32 && (uintptr_t)mask % 16 == 0;
    // column strips when the map is wide enough in rows and blocks to fill the GPU twice over; else one pixel per thread
    if (W <= 128) {
        const int groups = 128 / W, RB = groups * LS_R;
        const int row_blocks = (H + RB - 1) / RB;
        size_t smem_strip = sizeof(float) * (size_t)Cp * (24 + RB + 12);
        const int staged_strip = staged && smem_strip + sizeof(float) * (size_t)(RB * W * 9 + 4) <= 48 * 1024;
        if (staged_strip) smem_strip += sizeof(float) * (size_t)(RB * W * 9 + 4);
        if ((long long)row_blocks * B >= 296 && smem_strip <= 48 * 1024) {
            KAD_DISPATCH_DTYPE(dtype, {
                launch_pdl(lcsa_mask_strip_kernel<T>, dim3(row_blocks, B), 128, smem_strip, st, rowsum, A, Sm, w2, b2, w3, b3, mask, H, W, C, Cp, groups, mask_f32, rows_are_means, staged_strip);
            });
            KAD_CHECK_LAUNCH("lcsa_mask_from_partials (strips)");
            return KAD_OK;
        }
    }
    const int nrows = (127 / W + 2) < H ? (127 / W + 2) : H;
    const size_t smem = sizeof(float) * ((size_t)(2 * nrows + 1) * 12 * Cp + (staged ? 128 * 9 + 4 : 0));
    KAD_DISPATCH_DTYPE(dtype, {
        auto kern = lcsa_mask_flat_kernel<T>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "lcsa_mask smem attribute: %s", cudaGetErrorString(e));
        }
        launch_pdl(kern, dim3((H * W + 127) / 128, B), 128, smem, st, rowsum, A, Sm, w2, b2, w3, b3, mask, H, W, C, Cp, mask_f32, rows_are_means, staged);
    });
    KAD_CHECK_LAUNCH("lcsa_mask_from_partials");
    return KAD_OK;
}

// Shared memory of lcsa_fused_kernel for one branch; 0 if the branch does not qualify (W > 128: a block spans all columns).
static size_t lcsa_fused_smem(int H, int W, int C) {
    if (W > 128 || W < 1 || H < 1 || C < 1 || C > 256) return 0;
    const int Cp = (C + 3) & ~3, groups = 128 / W, P = groups * LS_R + 12;
    (void)H;
    return sizeof(float) * ((size_t)24 * Cp + (size_t)Cp * P + (size_t)2 * W * Cp + (size_t)W * C);
}

extern "C" int kad_lcsa_masks3_supported(int H, int W, int c0, int c1, int c2) {
    const int c[3] = {c0, c1, c2};
    for (int i = 0; i < 3; ++i) {
        const size_t s = lcsa_fused_smem(H >> i, W >> i, c[i]);
        if (s == 0 || s > 160 * 1024) return 0;
    }
    return 1;
}

extern "C" int kad_lcsa_masks3_from_partials(const float* const* rowpart, const float* const* colpart, int n_col_tiles, int n_row_groups,
                                             const float* const* w1, const float* const* b1, const float* const* bn_scale, const float* const* bn_shift,
                                             const float* const* w2, const float* const* b2, const float* const* w3, const float* const* b3,
                                             void* const* mask, int B, int H, int W, const int* c, int mask_f32, int dtype, void* stream) {
    KAD_CHECK_ARG(rowpart && colpart && w1 && b1 && bn_scale && bn_shift && w2 && b2 && w3 && b3 && mask && c, "kad_lcsa_masks3_from_partials: null pointer");
    KAD_CHECK_ARG(B > 0 && B <= 65535 && H >= 4 && W >= 4 && n_col_tiles > 0 && n_row_groups > 0, "kad_lcsa_masks3_from_partials: bad shape");
    if (!kad_lcsa_masks3_supported(H, W, c[0], c[1], c[2]))
        return fail(KAD_ERR_UNSUPPORTED, "kad_lcsa_masks3_from_partials: needs W <= 128 and the per-image operands in shared memory (W=%d, c=%d,%d,%d)", W, c[0], c[1], c[2]);
    LcsaFusedParams p{};
    p.nct = n_col_tiles; p.nrg = n_row_groups; p.mask_f32 = mask_f32;
    size_t smem = 0;
    int blocks = 0;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(rowpart[i] && colpart[i] && w1[i] && b1[i] && bn_scale[i] && bn_shift[i] && w2[i] && b2[i] && w3[i] && b3[i] && mask[i],
                      "kad_lcsa_masks3_from_partials: null pointer for branch %d", i);
        LcsaBranch& q = p.br[i];
        q.rowpart = rowpart[i]; q.colpart = colpart[i]; q.w1 = w1[i]; q.b1 = b1[i]; q.bn_m = bn_scale[i]; q.bn_a = bn_shift[i];
        q.w2 = w2[i]; q.b2 = b2[i]; q.w3 = w3[i]; q.b3 = b3[i]; q.mask = mask[i];
        q.H = H >> i; q.W = W >> i; q.C = c[i]; q.Cp = (c[i] + 3) & ~3; q.groups = 128 / q.W;
        const int RB = q.groups * LS_R;
        q.row_blocks = (q.H + RB - 1) / RB; q.first_block = blocks; blocks += q.row_blocks;
        const size_t s = lcsa_fused_smem(q.H, q.W, q.C);
        if (s > smem) smem = s;
    }
    cudaStream_t st = (cudaStream_t)stream;
    KAD_DISPATCH_DTYPE(dtype, {
        auto kern = lcsa_fused_kernel<T>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "lcsa_fused smem attribute: %s", cudaGetErrorString(e));
        }
        kern<<<dim3(blocks, B), 128, smem, st>>>(p);
    });
    KAD_CHECK_LAUNCH("lcsa_fused_kernel");
    return KAD_OK;
}

extern "C" int kad_se_excite(const float* gap_partial, int tiles, float inv_count,
                             const float* w1, const float* b1, const float* w2, const float* b2,
                             float* att, int B, int C, int Hd, void* stream) {
    KAD_CHECK_ARG(gap_partial && w1 && b1 && w2 && b2 && att, "kad_se_excite: null pointer");
    KAD_CHECK_ARG(B > 0 && C > 0 && Hd > 0 && tiles > 0, "kad_se_excite: bad shape");
    size_t smem = sizeof(float) * (size_t)(C + Hd + (C > 256 ? C : 256));
    KAD_CHECK_ARG(smem <= 48 * 1024, "kad_se_excite: C + hidden = %d too large", C + Hd);
    launch_pdl(se_excite_kernel, B, 256, smem, (cudaStream_t)stream, gap_partial, tiles, inv_count, w1, b1, w2, b2, att, C, Hd);
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
    const bool use_se = a->gap[0] != nullptr;
    const int out_ld = a->out_cstride ? a->out_cstride : a->C;
    KAD_CHECK_ARG(out_ld >= a->C, "kad_merge_upsample_residual: out_cstride %d < C %d", out_ld, a->C);
    MergeParams p;
    MergeSe se{};
    int hmax = 1;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(a->y[i] && a->h[i] > 0 && a->w[i] > 0 && a->c[i] > 0, "kad_merge_upsample_residual: bad branch %d", i);
        KAD_CHECK_ARG(a->att[i], "kad_merge_upsample_residual: att[%d] is null (with gap[] it is scratch of B * c floats)", i);
        p.y[i] = a->y[i]; p.att[i] = a->att[i]; p.c[i] = a->c[i]; p.h[i] = a->h[i]; p.w[i] = a->w[i];
        p.sy[i] = (float)a->h[i] / (float)a->H; p.sx[i] = (float)a->w[i] / (float)a->W;
        if (use_se) {
            KAD_CHECK_ARG(a->gap[i] && a->fc_w1[i] && a->fc_b1[i] && a->fc_w2[i] && a->fc_b2[i] && a->gap_tiles[i] > 0 && a->hidden[i] > 0,
                          "kad_merge_upsample_residual: incomplete squeeze-excite arguments for branch %d", i);
            se.gap[i] = a->gap[i]; se.w1[i] = a->fc_w1[i]; se.b1[i] = a->fc_b1[i]; se.w2[i] = a->fc_w2[i]; se.b2[i] = a->fc_b2[i];
            se.tiles[i] = a->gap_tiles[i]; se.hidden[i] = a->hidden[i]; se.inv[i] = 1.0f / (float)(a->h[i] * a->w[i]);
            if (a->hidden[i] > hmax) hmax = a->hidden[i];
        }
    }
    p.H = a->H; p.W = a->W; p.C = a->C;
    KAD_CHECK_ARG(a->B <= 65535, "kad_merge_upsample_residual: batch %d too large", a->B);
    cudaStream_t st = (cudaStream_t)stream;
    const int HW = a->H * a->W;
    const size_t se_smem = sizeof(float) * (size_t)(2 * a->C + 3 * hmax + 768);
    const bool vec8 = a->dtype != KAD_F32 && a->C % 8 == 0 && a->C <= 2048 && out_ld % 8 == 0 && (uintptr_t)a->x % 16 == 0 &&
                      (uintptr_t)a->out % 16 == 0 && se_smem <= 48 * 1024 && a->c[0] <= 256 && a->c[1] <= 256 && a->c[2] <= 256;
    // 16-bit tensors with C % 4 == 0: the column-walking kernel (no shared memory, attention read from att[])
    const bool col = a->dtype != KAD_F32 && a->C <= 1024 && a->c[0] >= 4 && a->c[1] >= 4 && a->c[2] >= 4 && (uintptr_t)a->x % 2 == 0 && (uintptr_t)a->out % 2 == 0;
    if (col) {
        if (use_se) {      // the attention takes its own small launches into att[] (callers that overlap them with other work pass gap = NULL)
            for (int i = 0; i < 3; ++i) {
                const int rc = kad_se_excite(a->gap[i], a->gap_tiles[i], se.inv[i], a->fc_w1[i], a->fc_b1[i], a->fc_w2[i], a->fc_b2[i],
                                             const_cast<float*>(a->att[i]), a->B, a->c[i], a->hidden[i], stream);
                if (rc) return rc;
            }
        }
        // alignment every channel group is guaranteed to have in x, out and its branch tensor
        int align = 8;
        while (align > 2 && ((uintptr_t)a->x % align || (uintptr_t)a->out % align || (a->C * 2) % align || (out_ld * 2) % align)) align >>= 1;
        int cbase = 0;
        for (int i = 0; i < 3; ++i) {
            while (align > 2 && ((uintptr_t)a->y[i] % align || (a->c[i] * 2) % align || (cbase * 2) % align)) align >>= 1;
            cbase += a->c[i];
        }
        const int C4 = (a->c[0] + 3) / 4 + (a->c[1] + 3) / 4 + (a->c[2] + 3) / 4;          // channel groups per pixel
        int PL = 256 / C4; if (PL > a->W) PL = a->W; if (PL < 1) PL = 1;
        const int xstrips = (a->W + PL - 1) / PL;
        // rows per block: long enough columns to amortise the per-thread set-up, enough blocks for a few waves
        int R = (int)(((long long)xstrips * a->H * a->B) / (148 * 8));
        R = R < 4 ? 4 : (R > 32 ? 32 : R);
        if (R > a->H) R = a->H;
        dim3 grid(xstrips, (a->H + R - 1) / R, a->B);
        KAD_CHECK_ARG(grid.y <= 65535, "kad_merge_upsample_residual: image too tall");
#define KAD_MERGE_COL(TT, AL) launch_pdl(merge_col_kernel<TT, AL>, grid, 256, 0, st, (const TT*)a->x, (TT*)a->out, p, C4, PL, R, out_ld)
        if (a->dtype == KAD_F16) { if (align == 8) KAD_MERGE_COL(__half, 8); else if (align == 4) KAD_MERGE_COL(__half, 4); else KAD_MERGE_COL(__half, 2); }
        else { if (align == 8) KAD_MERGE_COL(__nv_bfloat16, 8); else if (align == 4) KAD_MERGE_COL(__nv_bfloat16, 4); else KAD_MERGE_COL(__nv_bfloat16, 2); }
#undef KAD_MERGE_COL
        KAD_CHECK_LAUNCH("merge_col_kernel");
        return KAD_OK;
    }
    if (vec8) {
        const int G = a->C / 8, PL = 256 / G;
        const int se_floats = ((2 * a->C + 3 * hmax + 768 + 3) / 4) * 4;
        // rows per block for the staged kernel: enough blocks for two per SM, at most 16 rows, at most ~56 KB of shared memory
        auto stage_bytes = [&](int R, MergeStage* stg) {
            size_t o = 0;
            for (int i = 0; i < 3; ++i) {
                const bool same = a->h[i] == a->H && a->w[i] == a->W;
                int rows = same ? R : (int)((float)R * p.sy[i]) + 3;
                if (rows > a->h[i]) rows = a->h[i];
                if (stg) { stg->off[i] = (int)o; stg->cap_rows[i] = rows; }
                o += (((size_t)rows * a->w[i] * a->c[i] * 2 + 15) / 16) * 16 + 32;
            }
            if (stg) stg->tile_off = (int)o;
            return o + (size_t)R * a->W * (a->C + 2) * 2;
        };
        int R = (int)(((long long)a->H * a->B) / 296);
        R = R < 1 ? 1 : (R > 16 ? 16 : R);
        while (R > 1 && stage_bytes(R, nullptr) > 56 * 1024) --R;
        MergeStage stg{};
        const size_t sb = stage_bytes(R, &stg);
        bool aligned = true;
        for (int i = 0; i < 3; ++i) aligned = aligned && ((uintptr_t)a->y[i] % 4 == 0);
        if (sb + (size_t)se_floats * 4 <= 110 * 1024 && aligned) {
            const size_t smem = sb + (size_t)se_floats * 4;
            const bool pairs = a->c[0] % 2 == 0 && a->c[1] % 2 == 0 && a->c[2] % 2 == 0;
            dim3 grid((a->H + R - 1) / R, a->B);
#define KAD_MERGE_TILE(TT, PP)                                                                                          \
            {                                                                                                             \
                auto kern = merge_tile_kernel<TT, PP>;                                                                    \
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
                if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "merge smem attribute: %s", cudaGetErrorString(e));       \
                kern<<<grid, 256, smem, st>>>((const TT*)a->x, (uint4*)a->out, p, se, stg, use_se ? 1 : 0, R, out_ld / 8, se_floats); \
            }
            if (a->dtype == KAD_F16) { if (pairs) KAD_MERGE_TILE(__half, true) else KAD_MERGE_TILE(__half, false) }
            else { if (pairs) KAD_MERGE_TILE(__nv_bfloat16, true) else KAD_MERGE_TILE(__nv_bfloat16, false) }
#undef KAD_MERGE_TILE
            KAD_CHECK_LAUNCH("merge_tile_kernel");
            return KAD_OK;
        }
        long long want = ((long long)HW * a->B) / ((long long)PL * 148 * 8);
        const int iters = want < 2 ? 2 : (want > 16 ? 16 : (int)want);
        const int pix_per_block = iters * PL;
        dim3 grid((HW + pix_per_block - 1) / pix_per_block, a->B);
        if (a->dtype == KAD_F16)
            merge_vec8_kernel<__half><<<grid, 256, se_smem, st>>>((const uint4*)a->x, (uint4*)a->out, p, se, use_se ? 1 : 0, G, PL, pix_per_block, out_ld / 8);
        else
            merge_vec8_kernel<__nv_bfloat16><<<grid, 256, se_smem, st>>>((const uint4*)a->x, (uint4*)a->out, p, se, use_se ? 1 : 0, G, PL, pix_per_block, out_ld / 8);
        KAD_CHECK_LAUNCH("merge_vec8_kernel");
        return KAD_OK;
    }
    if (use_se) {      // general shapes: the attention takes its own small launches into the att[] scratch
        for (int i = 0; i < 3; ++i) {
            const int rc = kad_se_excite(a->gap[i], a->gap_tiles[i], se.inv[i], a->fc_w1[i], a->fc_b1[i], a->fc_w2[i], a->fc_b2[i],
                                         const_cast<float*>(a->att[i]), a->B, a->c[i], a->hidden[i], stream);
            if (rc) return rc;
        }
    }
    // two channels per thread (one 32-bit access) for 16-bit storage when every branch width is even
    const bool pairs = a->dtype != KAD_F32 && a->c[0] % 2 == 0 && a->c[1] % 2 == 0 && a->c[2] % 2 == 0 && out_ld % 2 == 0 &&
                       (uintptr_t)a->x % 4 == 0 && (uintptr_t)a->out % 4 == 0 && (uintptr_t)a->y[0] % 4 == 0 &&
                       (uintptr_t)a->y[1] % 4 == 0 && (uintptr_t)a->y[2] % 4 == 0;
    const int groups = pairs ? a->C / 2 : a->C;
    int Cp = 8;
    while (Cp < groups && Cp < 256) Cp <<= 1;          // channel groups per pixel lane, a power of two
    // pixels per thread: 4 on small feature maps (enough blocks to fill the GPU), up to 32 on large ones (amortises the
    // per-thread channel set-up)
    const int PL = 256 / Cp;
    long long want = ((long long)HW * a->B) / ((long long)PL * 148 * 8);
    int iters = want < 4 ? 4 : (want > 32 ? 32 : (int)want);
    int pix_per_block = iters * PL;
    dim3 grid((HW + pix_per_block - 1) / pix_per_block, a->B);
    if (pairs && a->dtype == KAD_F16) merge_kernel<__half, 2><<<grid, 256, 0, st>>>((const __half*)a->x, (__half*)a->out, p, Cp, pix_per_block, out_ld);
    else if (pairs) merge_kernel<__nv_bfloat16, 2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a->x, (__nv_bfloat16*)a->out, p, Cp, pix_per_block, out_ld);
    else {
        KAD_DISPATCH_DTYPE(a->dtype, {
            merge_kernel<T, 1><<<grid, 256, 0, st>>>((const T*)a->x, (T*)a->out, p, Cp, pix_per_block, out_ld);
        });
    }
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


namespace kad { namespace {
// 8 x 16-bit channels per thread (C % 8 == 0)
template <typename T>
__global__ void avg_pool_vec8_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int H, int W, int Ho, int Wo, int C8, int pool, size_t n) {
    const float inv = 1.f / (float)(pool * pool);
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % C8);
        size_t r = e / C8;
        const int xo = (int)(r % Wo); r /= Wo;
        const int yo = (int)(r % Ho); const int b = (int)(r / Ho);
        const uint4* base = x + (((size_t)b * H + yo * pool) * W + xo * pool) * C8 + c;
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int dy = 0; dy < pool; ++dy)
            for (int dx = 0; dx < pool; ++dx) {
                const uint4 v = base[((size_t)dy * W + dx) * C8];
                const T* h = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] += to_f<T>(h[i]);
            }
        uint4 o;
        T* ho = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) ho[i] = from_f<T>(s[i] * inv);
        y[e] = o;
    }
}
} }

extern "C" int kad_avg_pool(const void* x, void* y, int B, int H, int W, int C, int pool, int dtype, void* stream) {
    KAD_CHECK_ARG(x && y && B > 0 && H > 0 && W > 0 && C > 0, "kad_avg_pool: bad argument");
    KAD_CHECK_ARG(pool >= 1 && H / pool > 0 && W / pool > 0, "kad_avg_pool: pool %d leaves no output for %dx%d", pool, H, W);
    const int Ho = H / pool, Wo = W / pool;
    const size_t n = (size_t)B * Ho * Wo * C;
    if (dtype != KAD_F32 && C % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
        const size_t nv = n / 8;
        if (dtype == KAD_F16) avg_pool_vec8_kernel<__half><<<grid_for(nv, 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)y, H, W, Ho, Wo, C / 8, pool, nv);
        else avg_pool_vec8_kernel<__nv_bfloat16><<<grid_for(nv, 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)y, H, W, Ho, Wo, C / 8, pool, nv);
    } else {
        KAD_DISPATCH_DTYPE(dtype, {
            avg_pool_kernel<T><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const T*)x, (T*)y, H, W, Ho, Wo, C, pool, n);
        });
    }
    KAD_CHECK_LAUNCH("avg_pool_kernel");
    return KAD_OK;
}


// ------------------------------------------------------------------------------ detector glue kernels
namespace kad { namespace {

// 2x2 average pool with stride 1 (AConv's pre-pool, KAD-CNet/models/common.py:65): y[b,y,x,:] = mean of the 2x2 block at (y,x).
template <typename T>
__global__ void avg_pool2x2s1_vec8_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int H, int W, int C8, size_t n) {
    grid_dependency_wait(); grid_dependents_go();      // launched programmatically: nothing is read before the kernels in front are done
    const int Ho = H - 1, Wo = W - 1;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % C8);
        size_t r = e / C8;
        const int xo = (int)(r % Wo); r /= Wo;
        const int yo = (int)(r % Ho); const int b = (int)(r / Ho);
        const uint4* base = x + (((size_t)b * H + yo) * W + xo) * C8 + c;
        const uint4 v00 = base[0], v01 = base[C8], v10 = base[(size_t)W * C8], v11 = base[(size_t)(W + 1) * C8];
        const T* a = reinterpret_cast<const T*>(&v00); const T* bq = reinterpret_cast<const T*>(&v01);
        const T* cq = reinterpret_cast<const T*>(&v10); const T* d = reinterpret_cast<const T*>(&v11);
        uint4 o; T* ho = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) ho[i] = from_f<T>((to_f<T>(a[i]) + to_f<T>(bq[i]) + to_f<T>(cq[i]) + to_f<T>(d[i])) * 0.25f);
        y[e] = o;
    }
}
template <typename T>
__global__ void avg_pool2x2s1_kernel(const T* __restrict__ x, T* __restrict__ y, int H, int W, int C, size_t n) {
    const int Ho = H - 1, Wo = W - 1;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % C);
        size_t r = e / C;
        const int xo = (int)(r % Wo); r /= Wo;
        const int yo = (int)(r % Ho); const int b = (int)(r / Ho);
        const T* base = x + (((size_t)b * H + yo) * W + xo) * C + c;
        y[e] = from_f<T>((to_f<T>(base[0]) + to_f<T>(base[C]) + to_f<T>(base[(size_t)W * C]) + to_f<T>(base[(size_t)(W + 1) * C])) * 0.25f);
    }
}

__device__ __forceinline__ float silu_tanh(float v) { return silu_fast(v); }

// out[m][0..C) = act(y[m][0..C) + bias), 8 channels per thread; out rows are out_ld8 vectors apart (out may be y itself,
// or a channel slice of a wider tensor). Two vectors per thread are in flight.
template <typename T>
__global__ void __launch_bounds__(256)
bias_act_vec8_kernel(const uint4* __restrict__ y, uint4* __restrict__ out, const float* __restrict__ bias, unsigned C8, unsigned out_ld8,
                     unsigned long long n, int act) {
    grid_dependency_wait(); grid_dependents_go();      // launched programmatically: nothing is read before the kernels in front are done
    const unsigned long long stride = (unsigned long long)gridDim.x * 256;
    for (unsigned long long e0 = (unsigned long long)blockIdx.x * 256 + threadIdx.x; e0 < n; e0 += 2 * stride) {
        const unsigned long long e1 = e0 + stride;
        const bool two = e1 < n;
        uint4 v[2];
        v[0] = y[e0];
        if (two) v[1] = y[e1];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            if (k == 1 && !two) break;
            const unsigned long long e = k ? e1 : e0;
            const unsigned long long m = n <= 0xffffffffull ? (unsigned long long)((unsigned)e / C8) : e / C8;
            const unsigned c = (unsigned)(e - m * C8);
            T* h = reinterpret_cast<T*>(&v[k]);
            const float4 b0 = bias ? reinterpret_cast<const float4*>(bias)[2 * c] : make_float4(0, 0, 0, 0);
            const float4 b1 = bias ? reinterpret_cast<const float4*>(bias)[2 * c + 1] : make_float4(0, 0, 0, 0);
            const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = to_f<T>(h[i]) + bb[i];
                h[i] = from_f<T>(act == KAD_ACT_SILU ? silu_tanh(a) : (act == KAD_ACT_RELU ? fmaxf(a, 0.f) : a));
            }
            out[m * out_ld8 + c] = v[k];
        }
    }
}
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ y, T* __restrict__ out, const float* __restrict__ bias, int C, int out_ld, size_t n, int act) {
    grid_dependency_wait(); grid_dependents_go();      // launched programmatically: nothing is read before the kernels in front are done
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t m = e / C; const int c = (int)(e - m * C);
        const float a = to_f<T>(y[e]) + (bias ? bias[c] : 0.f);
        out[m * out_ld + c] = from_f<T>(apply_act(a, act));
    }
}

// out[b][y][x][0..C1) = low[b][y/2][x/2][:], out[b][y][x][C1..C1+C2) = skip[b][y][x][:]: nearest-neighbour 2x upsampling
// and channel concatenation in one pass, 8 channels per thread.
__global__ void __launch_bounds__(256)
upsample2x_concat_vec8_kernel(const uint4* __restrict__ low, const uint4* __restrict__ skip, uint4* __restrict__ out,
                              int h, int w, unsigned G1, unsigned G2, unsigned long long n) {
    grid_dependency_wait(); grid_dependents_go();      // launched programmatically: nothing is read before the kernels in front are done
    const unsigned G = G1 + G2;
    const int W = 2 * w;
    for (unsigned long long e = (unsigned long long)blockIdx.x * 256 + threadIdx.x; e < n; e += (unsigned long long)gridDim.x * 256) {
        const unsigned long long pix = e / G;                 // b*H*W + y*W + x
        const unsigned g = (unsigned)(e - pix * G);
        if (g >= G1) { out[e] = __ldg(skip + pix * G2 + (g - G1)); continue; }
        const unsigned long long row = pix / W;               // b*H + y
        const int x = (int)(pix - row * W);
        const unsigned long long bimg = row / (2 * h);
        const int y = (int)(row - bimg * 2 * h);
        out[e] = __ldg(low + ((bimg * h + (y >> 1)) * w + (x >> 1)) * G1 + g);
    }
}
template <typename T>
__global__ void upsample2x_concat_kernel(const T* __restrict__ low, const T* __restrict__ skip, T* __restrict__ out,
                                         int h, int w, int C1, int C2, size_t n) {
    const int C = C1 + C2, W = 2 * w;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t pix = e / C; const int c = (int)(e - pix * C);
        if (c >= C1) { out[e] = skip[pix * C2 + (c - C1)]; continue; }
        const size_t row = pix / W; const int x = (int)(pix - row * W);
        const size_t bimg = row / (2 * h); const int y = (int)(row - bimg * 2 * h);
        out[e] = low[((bimg * h + (y >> 1)) * w + (x >> 1)) * C1 + c];
    }
}

// uint8 NCHW image batch -> T NHWC, value * scale, channels zero-padded from C to Cp (Cp * sizeof(T) == 16 here)
template <typename T>
__global__ void image_to_nhwc_kernel(const unsigned char* __restrict__ img, T* __restrict__ y, int C, int Cp, size_t HW, size_t n, float scale) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t b = e / HW, p = e - b * HW;
        const unsigned char* src = img + b * C * HW + p;
        T* dst = y + e * Cp;
        for (int c = 0; c < Cp; ++c) dst[c] = from_f<T>(c < C ? (float)src[(size_t)c * HW] * scale : 0.f);
    }
}
} }

extern "C" int kad_avg_pool2x2s1(const void* x, void* y, int B, int H, int W, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(x && y && B > 0 && H > 1 && W > 1 && C > 0, "kad_avg_pool2x2s1: bad argument");
    const size_t n = (size_t)B * (H - 1) * (W - 1) * C;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != KAD_F32 && C % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
        const size_t nv = n / 8;
        if (dtype == KAD_F16) launch_pdl(avg_pool2x2s1_vec8_kernel<__half>, grid_for(nv, 256), 256, 0, st, (const uint4*)x, (uint4*)y, H, W, C / 8, nv);
        else launch_pdl(avg_pool2x2s1_vec8_kernel<__nv_bfloat16>, grid_for(nv, 256), 256, 0, st, (const uint4*)x, (uint4*)y, H, W, C / 8, nv);
    } else {
        KAD_DISPATCH_DTYPE(dtype, { avg_pool2x2s1_kernel<T><<<grid_for(n, 256), 256, 0, st>>>((const T*)x, (T*)y, H, W, C, n); });
    }
    KAD_CHECK_LAUNCH("avg_pool2x2s1_kernel");
    return KAD_OK;
}

extern "C" int kad_bias_act_to(const void* y, const float* bias, void* out, long long M, int C, int out_cstride, int act, int dtype, void* stream) {
    KAD_CHECK_ARG(y && out && M > 0 && C > 0, "kad_bias_act_to: bad argument");
    const int out_ld = out_cstride ? out_cstride : C;
    KAD_CHECK_ARG(out_ld >= C, "kad_bias_act_to: out_cstride %d < C %d", out_ld, C);
    const size_t n = (size_t)M * C;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != KAD_F32 && C % 8 == 0 && out_ld % 8 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0 && (!bias || (uintptr_t)bias % 16 == 0)) {
        const size_t nv = n / 8;
        size_t blocks = (nv + 511) / 512;
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (dtype == KAD_F16) launch_pdl(bias_act_vec8_kernel<__half>, (unsigned)blocks, 256, 0, st, (const uint4*)y, (uint4*)out, bias, C / 8, out_ld / 8, nv, act);
        else launch_pdl(bias_act_vec8_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, st, (const uint4*)y, (uint4*)out, bias, C / 8, out_ld / 8, nv, act);
    } else {
        KAD_DISPATCH_DTYPE(dtype, { launch_pdl(bias_act_kernel<T>, grid_for(n, 256), 256, 0, st, (const T*)y, (T*)out, bias, C, out_ld, n, act); });
    }
    KAD_CHECK_LAUNCH("bias_act_kernel");
    return KAD_OK;
}

extern "C" int kad_bias_act_inplace(void* y, const float* bias, long long M, int C, int act, int dtype, void* stream) {
    return kad_bias_act_to(y, bias, y, M, C, C, act, dtype, stream);
}

// ---- channel-slice copy: dst[m][dst_coff .. +C) = src[m][src_coff .. +C) for rows of different lengths --------------------------
namespace kad {
namespace {
template <typename V>
__global__ void __launch_bounds__(256)
copy_channels_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst, size_t nvec, unsigned vpr, unsigned vpr_magic, int exact,
                     size_t src_pitch, size_t dst_pitch) {
    grid_dependency_wait(); grid_dependents_go();      // launched programmatically: nothing is read before the kernels in front are done
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= nvec) return;
    // row = i / vpr: by multiplication with a rounded-up reciprocal when the index fits 32 bits, else by division
    const size_t m = exact ? (size_t)__umulhi((unsigned)i, vpr_magic) : i / vpr;
    const size_t v = i - m * vpr;
    *reinterpret_cast<V*>(dst + m * dst_pitch + v * sizeof(V)) = *reinterpret_cast<const V*>(src + m * src_pitch + v * sizeof(V));
}
}  // namespace
}  // namespace kad

extern "C" int kad_copy_channels(const void* src, int src_cstride, int src_coff, void* dst, int dst_cstride, int dst_coff,
                                 long long M, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(src && dst && M > 0 && C > 0, "kad_copy_channels: bad argument");
    KAD_CHECK_ARG(src_coff >= 0 && dst_coff >= 0 && src_coff + C <= src_cstride && dst_coff + C <= dst_cstride,
                  "kad_copy_channels: slice [%d, %d) / [%d, %d) outside rows of %d / %d channels", src_coff, src_coff + C, dst_coff, dst_coff + C, src_cstride, dst_cstride);
    KAD_CHECK_ARG(dtype == KAD_F32 || dtype == KAD_F16 || dtype == KAD_BF16, "kad_copy_channels: bad dtype");
    const size_t es = dtype == KAD_F32 ? 4 : 2;
    const unsigned char* s = (const unsigned char*)src + (size_t)src_coff * es;
    unsigned char* d = (unsigned char*)dst + (size_t)dst_coff * es;
    const size_t row = (size_t)C * es, sp = (size_t)src_cstride * es, dp = (size_t)dst_cstride * es;
    // widest vector that the row length, both row pitches and both first addresses allow
    const uintptr_t al = (uintptr_t)s | (uintptr_t)d | row | sp | dp;
    const int vb = !(al & 15) ? 16 : (!(al & 7) ? 8 : (!(al & 3) ? 4 : 2));
    const size_t vpr = row / vb, nvec = (size_t)M * vpr;
    KAD_CHECK_ARG((nvec + 255) / 256 <= 0x7fffffffull, "kad_copy_channels: too many elements");
    // floor(i * ceil(2^32 / vpr) / 2^32) == i / vpr whenever i * vpr < 2^32 (the rounding error of the reciprocal is below vpr / 2^32)
    const int exact = vpr > 1 && nvec <= 0xffffffffull / vpr;
    const unsigned magic = vpr > 1 ? (unsigned)((0x100000000ull + vpr - 1) / vpr) : 0u;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((nvec + 255) / 256);
    if (vb == 16) launch_pdl(copy_channels_kernel<uint4>, blocks, 256, 0, st, s, d, nvec, (unsigned)vpr, magic, exact, sp, dp);
    else if (vb == 8) launch_pdl(copy_channels_kernel<uint2>, blocks, 256, 0, st, s, d, nvec, (unsigned)vpr, magic, exact, sp, dp);
    else if (vb == 4) launch_pdl(copy_channels_kernel<uint32_t>, blocks, 256, 0, st, s, d, nvec, (unsigned)vpr, magic, exact, sp, dp);
    else launch_pdl(copy_channels_kernel<uint16_t>, blocks, 256, 0, st, s, d, nvec, (unsigned)vpr, magic, exact, sp, dp);
    KAD_CHECK_LAUNCH("copy_channels_kernel");
    return KAD_OK;
}

extern "C" int kad_upsample2x_concat(const void* low, const void* skip, void* out, int B, int h, int w, int C1, int C2, int dtype, void* stream) {
    KAD_CHECK_ARG(low && skip && out && B > 0 && h > 0 && w > 0 && C1 > 0 && C2 > 0, "kad_upsample2x_concat: bad argument");
    const size_t n = (size_t)B * 4 * h * w * (C1 + C2);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != KAD_F32 && C1 % 8 == 0 && C2 % 8 == 0 && (uintptr_t)low % 16 == 0 && (uintptr_t)skip % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const size_t nv = n / 8;
        launch_pdl(upsample2x_concat_vec8_kernel, grid_for(nv, 256), 256, 0, st, (const uint4*)low, (const uint4*)skip, (uint4*)out, h, w, C1 / 8, C2 / 8, nv);
    } else {
        KAD_DISPATCH_DTYPE(dtype, { upsample2x_concat_kernel<T><<<grid_for(n, 256), 256, 0, st>>>((const T*)low, (const T*)skip, (T*)out, h, w, C1, C2, n); });
    }
    KAD_CHECK_LAUNCH("upsample2x_concat_kernel");
    return KAD_OK;
}

extern "C" int kad_image_to_nhwc(const void* img_u8, void* y, int B, int C, int H, int W, int Cp, float scale, int dtype, void* stream) {
    KAD_CHECK_ARG(img_u8 && y && B > 0 && C > 0 && H > 0 && W > 0 && Cp >= C, "kad_image_to_nhwc: bad argument");
    const size_t HW = (size_t)H * W, n = (size_t)B * HW;
    KAD_DISPATCH_DTYPE(dtype, {
        image_to_nhwc_kernel<T><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const unsigned char*)img_u8, (T*)y, C, Cp, HW, n, scale);
    });
    KAD_CHECK_LAUNCH("image_to_nhwc_kernel");
    return KAD_OK;
}


// ---- SPPELAN pooling chain ------------------------------------------------------------------------------------------------
// y2 = maxpool5(y1), y3 = maxpool5(y2), y4 = maxpool5(y3) (kernel 5, stride 1, padding 2: SP of KAD-CNet/models/common.py:187-193
// as chained by SPPELAN.forward, :590-598) in one kernel that reads slice 0 of the concatenation [y1 | y2 | y3 | y4] and writes
// slices 1-3 in place, so neither the three pooled tensors nor the torch.cat exist as separate passes over memory.
// A block owns one image and 8 channels: the H x W plane of 16-byte vectors sits in shared memory and each pooling is a
// horizontal then a vertical running maximum over 5 (padding = the window simply stops at the border, as -inf padding does).
namespace kad {
namespace {
template <typename T> struct Vec2;
template <> struct Vec2<__half> { using type = __half2; };
template <> struct Vec2<__nv_bfloat16> { using type = __nv_bfloat162; };

template <typename T>
__device__ __forceinline__ uint4 max8(uint4 a, uint4 b) {
    using V = typename Vec2<T>::type;
    uint4 r;
    V* pr = reinterpret_cast<V*>(&r); const V* pa = reinterpret_cast<const V*>(&a); const V* pb = reinterpret_cast<const V*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = __hmax2_nan(pa[i], pb[i]);      // NaN propagates, as in the library's max pooling
    return r;
}

template <typename T>
__global__ void __launch_bounds__(256) spp_pool3_kernel(uint4* __restrict__ cat, int H, int W, int ld8, int c8) {
    extern __shared__ __align__(16) uint4 spp_sm[];
    uint4* a = spp_sm;                // current plane
    uint4* h = spp_sm + H * W;        // horizontally pooled plane
    const int b = blockIdx.y, ch = blockIdx.x, HW = H * W;
    uint4* base = cat + (size_t)b * HW * ld8 + ch;
    for (int e = threadIdx.x; e < HW; e += 256) a[e] = base[(size_t)e * ld8];
    __syncthreads();
    for (int pass = 1; pass <= 3; ++pass) {
        for (int e = threadIdx.x; e < HW; e += 256) {
            const int y = e / W, x = e - y * W;
            uint4 m = a[e];
#pragma unroll
            for (int d = -2; d <= 2; ++d) if (d != 0 && x + d >= 0 && x + d < W) m = max8<T>(m, a[e + d]);
            h[e] = m;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < HW; e += 256) {
            const int y = e / W;
            uint4 m = h[e];
#pragma unroll
            for (int d = -2; d <= 2; ++d) if (d != 0 && y + d >= 0 && y + d < H) m = max8<T>(m, h[e + d * W]);
            a[e] = m;
            base[(size_t)e * ld8 + (size_t)pass * c8] = m;
        }
        __syncthreads();
    }
}
}  // namespace
}  // namespace kad

extern "C" int kad_spp_pool3_supported(int H, int W, int C, int dtype) {
    return (dtype == KAD_F16 || dtype == KAD_BF16) && C > 0 && C % 8 == 0 && H > 0 && W > 0 && (size_t)H * W * 32 <= 200 * 1024;
}

extern "C" int kad_spp_pool3(void* cat, int B, int H, int W, int C, int dtype, void* stream) {
    KAD_CHECK_ARG(cat && B > 0 && B <= 65535, "kad_spp_pool3: bad argument");
    if (!kad_spp_pool3_supported(H, W, C, dtype))
        return fail(KAD_ERR_UNSUPPORTED, "kad_spp_pool3: needs f16/bf16, C %% 8 == 0 and a plane of H*W*32 bytes in shared memory (got H=%d W=%d C=%d)", H, W, C);
    KAD_CHECK_ARG((uintptr_t)cat % 16 == 0, "kad_spp_pool3: the tensor must be 16-byte aligned");
    const size_t smem = (size_t)H * W * 32;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(C / 8, B);
    if (dtype == KAD_F16) {
        auto kern = spp_pool3_kernel<__half>;
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                                if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "spp_pool3 smem attribute: %s", cudaGetErrorString(e)); }
        kern<<<grid, 256, smem, st>>>((uint4*)cat, H, W, 4 * C / 8, C / 8);
    } else {
        auto kern = spp_pool3_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                                if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "spp_pool3 smem attribute: %s", cudaGetErrorString(e)); }
        kern<<<grid, 256, smem, st>>>((uint4*)cat, H, W, 4 * C / 8, C / 8);
    }
    KAD_CHECK_LAUNCH("spp_pool3_kernel");
    return KAD_OK;
}
