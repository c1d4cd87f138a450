// Branch pyramid of a KAD-Conv layer in one pass over x: t_i = conv1x1_i(avg_pool_{2^i}(x)) + b_i for i = 0, 1, 2
// (KADConv.forward, KAD-Conv/kadconv/kad_conv.py:115 with convs[i][0]). The three projections read the same tensor; issued
// as three kernels x crosses HBM three times and each launch is latency-bound. Here a block stages a tile of 4 rows x
// TW columns of x in shared memory with asynchronous 16-byte copies (everything in flight at once), forms the 2x2 and
// 4x4 averages from the staged tile (rounded to the storage type, as the reference's avg_pool2d output is), runs the three
// 1x1 convolutions on the warp-level tensor-core instruction (fp32 accumulation) and writes the three result tiles as
// contiguous row segments.
#include "kad_mma.cuh"

namespace kad {
namespace {

struct PyramidParams {
    const void* x; const float* w[3]; const float* b[3]; void* t[3];
    int B, H, W, dim, c[3];
    int TW, KC, xpitch;           // tile width (a multiple of 4), 16-channel chunks, bytes per staged pixel (dim*2 + 16)
    unsigned vpp_magic;           // ceil(2^32 / (dim / 8)): n / (dim / 8) == __umulhi(n, vpp_magic) for the index ranges used here
    int off_p1, off_p2, off_B, off_bias, off_out, off_colacc, off_part;   // shared-memory byte offsets
    // optional by-products for the LCSA that follows (kad_conv.py:27-28: means over rows and over columns of every t_i):
    // rowpart[i] [B][h_i][gridDim.x][c_i]: sum over the columns of this block's tile; colpart[i] [B][gridDim.y][w_i][c_i]:
    // sum over the rows this block covers (RT consecutive 4-row tiles); sums of the values as stored (rounded to T)
    float* rowpart[3]; float* colpart[3];
    int RT;
    // optional LCSA preparation in the tail (set counters): see lcsa_prepare_image
    int* counters;
    const float* lw1[3]; const float* lb1[3]; const float* lbn_m[3]; const float* lbn_a[3];
    float* l_rowmean[3]; float* l_A[3]; float* l_Sm[3];
};

// First, separable stage of one branch's LCSA for image b, from the partial sums every block of the image has written:
// row means (sums over the column tiles, / W), column sums (over the row groups), then per column w and channel c
//   A[b][w][c] = (sum_k w1[c][k] * colmean[w + k - 5][c] + b1[c]) * bn_m[c] + bn_a[c],   Sm[w][c] = (sum of the taps inside the row) * bn_m[c]
// (the 1x11 convolution of rowmean[h] + colmean[w] separates into rowmean[h] * S[w] + conv(colmean)[w]; zero padding makes S
// depend on w). Same arithmetic and summation order as lcsa_prep_partials_kernel, which does this in a launch of its own.
// One block, all threads; partial sums are read past L1 (other blocks wrote them). colsum_s: W*C floats of shared memory.
__device__ void lcsa_prepare_image(const float* rowpart, int nct, const float* colpart, int nrg,
                                   const float* __restrict__ w1, const float* __restrict__ b1, const float* __restrict__ bn_m, const float* __restrict__ bn_a,
                                   float* __restrict__ A, float* __restrict__ Sm, float* __restrict__ rowmean,
                                   int b, int H, int W, int C, float* colsum_s, int tid) {
    const int Cp = (C + 3) & ~3;
    const float invW = 1.f / (float)W;
    const float* cp = colpart + (size_t)b * nrg * W * C;
    for (int e = tid; e < W * C; e += MMA_THREADS) {
        float s = 0.f;
        for (int g = 0; g < nrg; ++g) s += __ldcg(cp + (size_t)g * W * C + e);
        colsum_s[e] = s;
    }
    for (int e = tid; e < H * C; e += MMA_THREADS) {
        const int h = e / C, c = e - h * C;
        float s = 0.f;
        for (int k = 0; k < nct; ++k) s += __ldcg(rowpart + (((size_t)b * H + h) * nct + k) * C + c);
        rowmean[((size_t)b * H + h) * C + c] = s * invW;
    }
    __syncthreads();
    const float invH = 1.f / (float)H;
    for (int e = tid; e < W * Cp; e += MMA_THREADS) {
        const int w = e / Cp, c = e - w * Cp;
        float av = 0.f, sv = 0.f;
        if (c < C) {
            float conv = 0.f, S = 0.f;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                const int ww = w + k - 5;
                if (ww >= 0 && ww < W) {
                    const float wk = w1[c * 11 + k];
                    conv = fmaf(wk, colsum_s[ww * C + c] * invH, conv);
                    S += wk;
                }
            }
            const float m = bn_m[c];
            av = (conv + b1[c]) * m + bn_a[c]; sv = S * m;
        }
        A[((size_t)b * W + w) * Cp + c] = av;
        if (b == 0) Sm[(size_t)w * Cp + c] = sv;
    }
    __syncthreads();
}

// Weight fragments of a 1x1 convolution w[Cout][Cin] (see stage_weights of the deformable kernel for the slot layout).
template <typename T>
__device__ __forceinline__ void stage_weights_1x1(uint2* dst, const float* __restrict__ w, int Cin, int Cout, int KC, int NT, int tid, int nthreads = MMA_THREADS) {
    for (int e = tid; e < KC * NT * 32; e += nthreads) {
        const int lane = e & 31, f = e >> 5, nt = f % NT, kc = f / NT;
        const int n = nt * 8 + (lane >> 2), t = lane & 3, ch = kc * 16 + 4 * t;
        const int first = lane_first_channel(kc, t, Cin);
        float v[4];
        if (n < Cout && first == ch && !(Cin & 3) && !(reinterpret_cast<uintptr_t>(w) & 15)) {      // the lane's four channels exist: one 16-byte load
            const float4 q = __ldg(reinterpret_cast<const float4*>(w + (size_t)n * Cin + ch));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = first + j;
                v[j] = (n < Cout && c >= ch && c < Cin) ? w[(size_t)n * Cin + c] : 0.f;
            }
        }
        dst[e] = make_uint2(pack2<T>(v[0], v[1]), pack2<T>(v[2], v[3]));
    }
}

template <typename T> __device__ __forceinline__ float2 up2(uint32_t u);
template <> __device__ __forceinline__ float2 up2<__half>(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
template <> __device__ __forceinline__ float2 up2<__nv_bfloat16>(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }

// mean of the N x N staged pixels whose top-left corner is s (rows `rowpitch` bytes apart, pixels `xp` bytes apart), for 8
// channels: summed in fp32, rounded once (as F.avg_pool2d rounds its output)
template <typename T, int N>
__device__ __forceinline__ uint4 mean_block(const unsigned char* s, int xp, size_t rowpitch) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int r = 0; r < N; ++r)
#pragma unroll
        for (int c = 0; c < N; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(s + r * rowpitch + (size_t)c * xp);
            const uint32_t* pv = &v.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = up2<T>(pv[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
        }
    const float inv = 1.f / (float)(N * N);
    uint4 out; uint32_t* po = &out.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) po[i] = pack2<T>(acc[2 * i] * inv, acc[2 * i + 1] * inv);
    return out;
}

template <typename T, int NT>
__global__ void __launch_bounds__(MMA_THREADS)
pyramid_project_kernel(const PyramidParams p) {
    extern __shared__ __align__(16) unsigned char sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int TW = p.TW, dim = p.dim, KC = p.KC, xp = p.xpitch;
    const int b = blockIdx.z, c0 = blockIdx.x * TW;
    const int cols = min(TW, p.W - c0);
    unsigned char* xt = sm;                                   // [4][TW] pixels of xp bytes
    unsigned char* p1 = sm + p.off_p1;                        // [2][TW/2]
    unsigned char* p2 = sm + p.off_p2;                        // [1][TW/4]
    uint2* Bs = reinterpret_cast<uint2*>(sm + p.off_B);       // [3][KC][NT][32]
    float* bias = reinterpret_cast<float*>(sm + p.off_bias);  // [3][NT*8]
    unsigned char* outs = sm + p.off_out;                     // result tiles of the three branches, one after the other
    float* colacc = reinterpret_cast<float*>(sm + p.off_colacc);   // column sums of the three result tiles over this block's row tiles
    float* part = reinterpret_cast<float*>(sm + p.off_part);       // [768] partial row sums
    const bool sums = p.rowpart[0] != nullptr;
    const int ncolacc = TW * p.c[0] + (TW >> 1) * p.c[1] + (TW >> 2) * p.c[2];
    if (sums) for (int e = tid; e < ncolacc; e += MMA_THREADS) colacc[e] = 0.f;

    const int vpp = dim >> 3;                                 // 16-byte vectors per pixel
    const unsigned char* xb = reinterpret_cast<const unsigned char*>(p.x) + (size_t)b * p.H * p.W * dim * 2;
    // asynchronous copy of row tile `rt` of this block into xt (nothing if the tile lies below the image)
    auto stage_x = [&](int rt) {
        const int r0 = (blockIdx.y * p.RT + rt) * 4;
        const int rows = min(4, p.H - r0);
        for (int r = 0; r < rows; ++r) {          // a tile row is one contiguous run of cols * dim * 2 bytes in x
            const unsigned char* src = xb + ((size_t)(r0 + r) * p.W + c0) * dim * 2;
            unsigned char* dst = xt + (size_t)r * TW * xp;
            for (int v = tid; v < cols * vpp; v += MMA_THREADS) {
                const int c = (int)__umulhi((unsigned)v, p.vpp_magic), k = v - c * vpp;
                cp_async16(dst + (size_t)c * xp + 16 * k, src + 16 * (size_t)v);
            }
        }
    };
    stage_x(0);
    for (int rt = 0; rt < p.RT; ++rt) {
    const int r0 = (blockIdx.y * p.RT + rt) * 4;
    if (r0 >= p.H) break;
    // ---- x is on its way (asynchronous); weights and bias meanwhile --------------------------------------------------
    if (rt == 0) {
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            stage_weights_1x1<T>(Bs + i * KC * NT * 32, p.w[i], dim, p.c[i], KC, NT, tid);
            for (int e = tid; e < NT * 8; e += MMA_THREADS) bias[i * NT * 8 + e] = (e < p.c[i] && p.b[i]) ? p.b[i][e] : 0.f;
        }
    }
    cp_async_wait_all();
    __syncthreads();

    // ---- 2x2 and 4x4 means (only where all contributing pixels exist: floor-mode pooling) -----------------------------
    const int h1 = p.H >> 1, w1 = p.W >> 1, h2 = p.H >> 2, w2 = p.W >> 2;
    const int TW1 = TW >> 1, TW2 = TW >> 2;
    for (int v = tid; v < 2 * TW1 * vpp; v += MMA_THREADS) {
        const int px = (int)__umulhi((unsigned)v, p.vpp_magic), k = v - px * vpp, r = px >= TW1 ? 1 : 0, c = px - r * TW1;
        if ((r0 >> 1) + r < h1 && (c0 >> 1) + c < w1) {
            *reinterpret_cast<uint4*>(p1 + (size_t)px * xp + 16 * k) = mean_block<T, 2>(xt + (size_t)((2 * r) * TW + 2 * c) * xp + 16 * k, xp, (size_t)TW * xp);
        }
    }
    for (int v = tid; v < TW2 * vpp; v += MMA_THREADS) {
        const int c = (int)__umulhi((unsigned)v, p.vpp_magic), k = v - c * vpp;
        if ((r0 >> 2) < h2 && (c0 >> 2) + c < w2)
            *reinterpret_cast<uint4*>(p2 + (size_t)c * xp + 16 * k) = mean_block<T, 4>(xt + (size_t)(4 * c) * xp + 16 * k, xp, (size_t)TW * xp);
    }
    __syncthreads();

    // ---- the three 1x1 convolutions: 16-pixel tiles of [x tile | 2x2 means | 4x4 means] -------------------------------
    const int n0 = (4 * TW + 15) >> 4, n1 = (2 * TW1 + 15) >> 4, n2 = (TW2 + 15) >> 4;
    int obase[3]; obase[0] = 0; obase[1] = 4 * TW * p.c[0] * 2; obase[2] = obase[1] + 2 * TW1 * p.c[1] * 2;
    for (int mt = warp; mt < n0 + n1 + n2; mt += MMA_THREADS / 32) {
        const int i = mt < n0 ? 0 : (mt < n0 + n1 ? 1 : 2);
        const int m0 = (i == 0 ? mt : (i == 1 ? mt - n0 : mt - n0 - n1)) * 16;
        const int npx = i == 0 ? 4 * TW : (i == 1 ? 2 * TW1 : TW2), ci = i == 0 ? p.c[0] : (i == 1 ? p.c[1] : p.c[2]);
        const unsigned char* src = i == 0 ? xt : (i == 1 ? p1 : p2);
        const uint2* Bi = Bs + i * KC * NT * 32;
        const int rlo = min(m0 + g, npx - 1), rhi = min(m0 + g + 8, npx - 1);   // (rows past the end repeat the last pixel, never stored)
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
#pragma unroll 1
        for (int kc = 0; kc < KC; ++kc) {
            const int coff = 2 * lane_first_channel(kc, t, dim);
            const uint2 lo = *reinterpret_cast<const uint2*>(src + (size_t)rlo * xp + coff);
            const uint2 hi = *reinterpret_cast<const uint2*>(src + (size_t)rhi * xp + coff);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma16816<T>(acc[nt], lo.x, hi.x, lo.y, hi.y, Bi[(kc * NT + nt) * 32 + lane]);
        }
        T* ot = reinterpret_cast<T*>(outs + (i == 0 ? obase[0] : (i == 1 ? obase[1] : obase[2])));
        const float* bi = bias + i * NT * 8;
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int px = m0 + g + 8 * hrow;
            if (px >= npx) continue;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int co = nt * 8 + 2 * t;
                if (co >= ci) continue;
                const float v0 = acc[nt][2 * hrow] + bi[co], v1 = acc[nt][2 * hrow + 1] + bi[co + 1];
                T* o = ot + (size_t)px * ci + co;
                if (!(ci & 1)) *reinterpret_cast<uint32_t*>(o) = pack2<T>(v0, v1);
                else { o[0] = from_f<T>(v0); if (co + 1 < ci) o[1] = from_f<T>(v1); }
            }
        }
    }
    __syncthreads();
    if (rt + 1 < p.RT) stage_x(rt + 1);       // xt and the pooled tiles are consumed: the next tile loads during the copy-out and the sums

    // ---- result tiles -> global, row segment by row segment (contiguous) ---------------------------------------------
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int ci = p.c[i], tw = TW >> i, hi_ = p.H >> i, wi = p.W >> i;
        const int rr0 = r0 >> i, cc0 = c0 >> i, nrows = min(4 >> i, hi_ - rr0), ncols = min(tw, wi - cc0);
        if (nrows <= 0 || ncols <= 0) continue;
        const T* ot = reinterpret_cast<const T*>(outs + obase[i]);
        T* dst = reinterpret_cast<T*>(p.t[i]) + (((size_t)b * hi_ + rr0) * wi + cc0) * ci;
        const int seg = ncols * ci;                           // elements per row segment
        // widest access that every row segment's length, its source in shared memory and its destination allow
        const uintptr_t al = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(ot) | (uintptr_t)(2 * seg) | (uintptr_t)(2 * wi * ci) | (uintptr_t)(2 * tw * ci);
        for (int r = 0; r < nrows; ++r) {
            const T* srow = ot + (size_t)r * tw * ci;
            T* drow = dst + (size_t)r * wi * ci;
            if (!(al & 15)) { for (int k = tid; k < (seg >> 3); k += MMA_THREADS) reinterpret_cast<uint4*>(drow)[k] = reinterpret_cast<const uint4*>(srow)[k]; }
            else if (!(al & 7)) { for (int k = tid; k < (seg >> 2); k += MMA_THREADS) reinterpret_cast<uint2*>(drow)[k] = reinterpret_cast<const uint2*>(srow)[k]; }
            else if (!(al & 3)) { for (int k = tid; k < (seg >> 1); k += MMA_THREADS) reinterpret_cast<uint32_t*>(drow)[k] = reinterpret_cast<const uint32_t*>(srow)[k]; }
            else { for (int k = tid; k < seg; k += MMA_THREADS) drow[k] = srow[k]; }
        }
    }

    // ---- by-products: sums over the tile's columns (per row) and rows (per column), in a fixed order ----------------------
    if (sums) {
        int cabase = 0, pbase = 0;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int ci = p.c[i], tw = TW >> i, hi_ = p.H >> i, wi = p.W >> i;
            const int rr0 = r0 >> i, cc0 = c0 >> i, nrows = max(0, min(4 >> i, hi_ - rr0)), ncols = max(0, min(tw, wi - cc0));
            const T* ot = reinterpret_cast<const T*>(outs + obase[i]);
            for (int e = tid; e < ncols * ci; e += MMA_THREADS) {          // e = col*ci + c: consecutive addresses of a tile row
                float a = 0.f;
                for (int r = 0; r < nrows; ++r) a += to_f<T>(ot[(size_t)r * tw * ci + e]);
                colacc[cabase + e] += a;
            }
            // row sums: Q threads per (row, channel), each over every Q-th column
            const int nrc = nrows * ci, Q = nrc > 0 ? max(1, min(8, 256 / nrc)) : 1;
            for (int e = tid; e < nrc * Q; e += MMA_THREADS) {
                const int q = e / nrc, rc = e - q * nrc, r = rc / ci, c = rc - r * ci;
                float a = 0.f;
                for (int col = q; col < ncols; col += Q) a += to_f<T>(ot[((size_t)r * tw + col) * ci + c]);
                part[pbase + e] = a;
            }
            cabase += tw * ci; pbase += 256;
        }
        __syncthreads();
        pbase = 0;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int ci = p.c[i], hi_ = p.H >> i, rr0 = r0 >> i, nrows = max(0, min(4 >> i, hi_ - rr0));
            const int nrc = nrows * ci, Q = nrc > 0 ? max(1, min(8, 256 / nrc)) : 1;
            for (int rc = tid; rc < nrc; rc += MMA_THREADS) {
                float a = 0.f;
                for (int q = 0; q < Q; ++q) a += part[pbase + q * nrc + rc];
                const int r = rc / ci, c = rc - r * ci;
                p.rowpart[i][(((size_t)b * hi_ + rr0 + r) * gridDim.x + blockIdx.x) * ci + c] = a;
            }
            pbase += 256;
        }
    }
    }   // row tiles

    if (sums) {
        __syncthreads();
        int cabase = 0;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int ci = p.c[i], tw = TW >> i, wi = p.W >> i, cc0 = c0 >> i, ncols = max(0, min(tw, wi - cc0));
            for (int e = tid; e < ncols * ci; e += MMA_THREADS)
                p.colpart[i][(((size_t)b * gridDim.y + blockIdx.y) * wi + cc0) * ci + e] = colacc[cabase + e];
            cabase += tw * ci;
        }
    }

    // ---- LCSA preparation by whichever block finishes this image last ----------------------------------------------------
    if (p.counters) {
        __shared__ int s_last;
        __threadfence();                                      // this block's partial sums are visible device-wide ...
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(p.counters + b, 1) == (int)(gridDim.x * gridDim.y) - 1;     // ... before it is counted
        __syncthreads();
        if (s_last) {
            __threadfence();
            float* colsum_s = reinterpret_cast<float*>(sm);   // everything staged in shared memory is dead by now
#pragma unroll 1
            for (int i = 0; i < 3; ++i)
                lcsa_prepare_image(p.rowpart[i], gridDim.x, p.colpart[i], gridDim.y, p.lw1[i], p.lb1[i], p.lbn_m[i], p.lbn_a[i],
                                   p.l_A[i], p.l_Sm[i], p.l_rowmean[i], b, p.H >> i, p.W >> i, p.c[i], colsum_s, tid);
            if (tid == 0) p.counters[b] = 0;                  // ready for the next launch
        }
    }
}

// ---- the same three projections by warps that own column segments ------------------------------------------------------------------
// A block covers PC_COLS columns of x and RG rows of one image; a warp owns one 16-pixel segment of ONE branch (8 + 4 + 2 segments
// for 128 columns) and walks down the rows of the group. Its A fragments come straight from global memory (a quarter-warp reads the
// 32 contiguous bytes of a pixel's 16-channel chunk: every sector is used in full; for a pooled branch the lane averages the 2x2 or
// 4x4 pixels in the order and with the rounding of the staged kernel above), the results leave from the accumulators, and the
// by-products need no second pass: column sums accumulate in the registers that hold the accumulator layout (same lane = same
// column in every row), row sums are a butterfly over the eight pixel lanes plus one small reduction over the segments at the end
// of the block. No shared-memory tile of x, no barrier between rows; x is read once from HBM and, for the pooled branches, again
// from L2 / L1. Outputs are bit-identical to the staged kernel's (same contraction order); the partial sums differ in summation order.
constexpr int PC_COLS = 128;

struct ColsPlan { int nct, RT, nrg, S[3], warps; size_t smem; };

template <typename T, int P>
__device__ __forceinline__ uint2 pooled8(const unsigned char* p, size_t rowbytes, int pixbytes) {
    if (P == 1) return ldg8<8>(p);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < P; ++r) {
        uint2 v[P];
#pragma unroll
        for (int c = 0; c < P; ++c) v[c] = ldg8<8>(p + r * rowbytes + c * pixbytes);
#pragma unroll
        for (int c = 0; c < P; ++c) {
            const float2 a = up2<T>(v[c].x), b = up2<T>(v[c].y);
            acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        }
    }
    const float inv = 1.f / (float)(P * P);
    return make_uint2(pack2<T>(acc[0] * inv, acc[1] * inv), pack2<T>(acc[2] * inv, acc[3] * inv));
}

// one warp's rows of branch I (pooling factor P = 2^I)
template <typename T, int NT, int P>
__device__ __forceinline__ void cols_branch(const PyramidParams& p, const uint2* __restrict__ Bi, const float* __restrict__ bias_i, float* __restrict__ rowseg_i,
                                            int i, int s, int nseg, int RG, int nct, int nrg, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, rg = blockIdx.y, ct = blockIdx.x;
    const int hi = p.H >> i, wi = p.W >> i, ci = p.c[i], KC = p.KC, dim = p.dim;
    const int tile_lo = (ct * PC_COLS) >> i, tile_hi = min(wi, ((ct + 1) * PC_COLS) >> i);
    const int col0 = tile_lo + 16 * s;
    if (col0 >= tile_hi) return;                                     // this tile has fewer segments than the widest one
    const bool ok_lo = col0 + g < tile_hi, ok_hi = col0 + g + 8 < tile_hi;
    const int cl = min(col0 + g, tile_hi - 1), ch = min(col0 + g + 8, tile_hi - 1);      // lanes past the end re-read the last pixel, never stored
    const int rgi = RG >> i, r_begin = rg * rgi, r_end = min(hi, r_begin + rgi);
    const int pix = dim * 2;
    const size_t rowbytes = (size_t)p.W * pix;
    const bool sums = p.rowpart[0] != nullptr, pairs = !(ci & 1);
    T* tb = reinterpret_cast<T*>(p.t[i]);
    float colsum[NT][4], bz[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) colsum[nt][j] = 0.f;
        const int co = nt * 8 + 2 * t;
        bz[nt][0] = co < ci ? bias_i[co] : 0.f; bz[nt][1] = co + 1 < ci ? bias_i[co + 1] : 0.f;
    }
    constexpr int KC_UNROLL = P == 1 ? 2 : 1;       // 16-channel chunks whose loads are in flight together (4 / 8 / 32 loads per lane; deeper measured no faster)
    // rows per trip. Two rows at once double the loads a warp has in flight, but the 28 registers they cost take a block off
    // every SM at the detector's widths, and the forward measured 2 % slower: one row.
    constexpr int RPT = 1;
    for (int r = r_begin; r < r_end; r += RPT) {
        const unsigned char* base[RPT];
        float acc[RPT][NT][4];
#pragma unroll
        for (int q = 0; q < RPT; ++q) {
            const int rr = min(r + q, r_end - 1);                    // a row past the end repeats the last one, never stored
            base[q] = reinterpret_cast<const unsigned char*>(p.x) + ((size_t)b * p.H + (size_t)P * rr) * rowbytes;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[q][nt][j] = 0.f;
        }
#pragma unroll KC_UNROLL
        for (int kc = 0; kc < KC; ++kc) {
            const int coff = 2 * lane_first_channel(kc, t, dim);
            uint2 lo[RPT], hv[RPT];
#pragma unroll
            for (int q = 0; q < RPT; ++q) {
                lo[q] = pooled8<T, P>(base[q] + (size_t)(P * cl) * pix + coff, rowbytes, pix);
                hv[q] = pooled8<T, P>(base[q] + (size_t)(P * ch) * pix + coff, rowbytes, pix);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint2 bf = Bi[(kc * NT + nt) * 32 + lane];
#pragma unroll
                for (int q = 0; q < RPT; ++q) mma16816<T>(acc[q][nt], lo[q].x, hv[q].x, lo[q].y, hv[q].y, bf);
            }
        }
#pragma unroll
        for (int q = 0; q < RPT; ++q) {
            if (r + q >= r_end) break;
            T* trow = tb + ((size_t)b * hi + r + q) * wi * ci;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int co = nt * 8 + 2 * t;
                const bool c0ok = co < ci, c1ok = co + 1 < ci;
                const float b0 = bz[nt][0], b1 = bz[nt][1];
                const uint32_t ulo = pack2<T>(acc[q][nt][0] + b0, acc[q][nt][1] + b1), uhi = pack2<T>(acc[q][nt][2] + b0, acc[q][nt][3] + b1);
                if (c0ok) {
                    if (pairs) {
                        if (ok_lo) *reinterpret_cast<uint32_t*>(trow + (size_t)cl * ci + co) = ulo;
                        if (ok_hi) *reinterpret_cast<uint32_t*>(trow + (size_t)ch * ci + co) = uhi;
                    } else {
                        uint16_t* o = reinterpret_cast<uint16_t*>(trow);
                        if (ok_lo) { o[(size_t)cl * ci + co] = (uint16_t)ulo; if (c1ok) o[(size_t)cl * ci + co + 1] = (uint16_t)(ulo >> 16); }
                        if (ok_hi) { o[(size_t)ch * ci + co] = (uint16_t)uhi; if (c1ok) o[(size_t)ch * ci + co + 1] = (uint16_t)(uhi >> 16); }
                    }
                }
                if (sums) {                                          // of the values as stored (rounded to T)
                    const float2 flo = up2<T>(ulo), fhi = up2<T>(uhi);
                    const float l0 = (ok_lo && c0ok) ? flo.x : 0.f, l1 = (ok_lo && c1ok) ? flo.y : 0.f;
                    const float h0 = (ok_hi && c0ok) ? fhi.x : 0.f, h1 = (ok_hi && c1ok) ? fhi.y : 0.f;
                    colsum[nt][0] += l0; colsum[nt][1] += l1; colsum[nt][2] += h0; colsum[nt][3] += h1;
                    float rs0 = l0 + h0, rs1 = l1 + h1;
#pragma unroll
                    for (int m = 4; m < 32; m <<= 1) { rs0 += __shfl_xor_sync(0xffffffffu, rs0, m); rs1 += __shfl_xor_sync(0xffffffffu, rs1, m); }
                    if (g == 0) {
                        float* rsq = rowseg_i + ((size_t)(r + q - r_begin) * nseg + s) * (NT * 8) + co;
                        rsq[0] = rs0; rsq[1] = rs1;
                    }
                }
            }
        }
    }
    if (sums) {
        float* cp = p.colpart[i] + ((size_t)b * nrg + rg) * wi * ci;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int co = nt * 8 + 2 * t;
            if (co < ci) {
                if (ok_lo) { cp[(size_t)cl * ci + co] = colsum[nt][0]; if (co + 1 < ci) cp[(size_t)cl * ci + co + 1] = colsum[nt][1]; }
                if (ok_hi) { cp[(size_t)ch * ci + co] = colsum[nt][2]; if (co + 1 < ci) cp[(size_t)ch * ci + co + 1] = colsum[nt][3]; }
            }
        }
    }
}

template <typename T, int NT>
__global__ void __launch_bounds__(448)
pyramid_cols_kernel(const PyramidParams p, int S0, int S1, int S2, int RG, int nct, int nrg) {
    extern __shared__ __align__(16) unsigned char sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int KC = p.KC;
    uint2* Bs = reinterpret_cast<uint2*>(sm);                                  // [3][KC][NT][32]
    float* bias = reinterpret_cast<float*>(sm + (size_t)3 * KC * NT * 32 * 8);  // [3][NT*8]
    float* rowseg0 = bias + 3 * NT * 8;                                        // branch i: [RG >> i][S_i][NT*8]
    float* rowseg1 = rowseg0 + (size_t)RG * S0 * NT * 8;
    float* rowseg2 = rowseg1 + (size_t)(RG >> 1) * S1 * NT * 8;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        stage_weights_1x1<T>(Bs + i * KC * NT * 32, p.w[i], p.dim, p.c[i], KC, NT, tid, nthreads);
        for (int e = tid; e < NT * 8; e += nthreads) bias[i * NT * 8 + e] = (e < p.c[i] && p.b[i]) ? p.b[i][e] : 0.f;
    }
    grid_dependency_wait();              // weights and bias are parameters; x comes from the kernel before
    grid_dependents_go();
    __syncthreads();
    if (warp < S0) cols_branch<T, NT, 1>(p, Bs, bias, rowseg0, 0, warp, S0, RG, nct, nrg, lane);
    else if (warp < S0 + S1) cols_branch<T, NT, 2>(p, Bs + KC * NT * 32, bias + NT * 8, rowseg1, 1, warp - S0, S1, RG, nct, nrg, lane);
    else cols_branch<T, NT, 4>(p, Bs + 2 * KC * NT * 32, bias + 2 * NT * 8, rowseg2, 2, warp - S0 - S1, S2, RG, nct, nrg, lane);
    if (p.rowpart[0] == nullptr) return;
    __syncthreads();
    // row sums over the segments this block's tile really has, in segment order
    const int b = blockIdx.z, rg = blockIdx.y, ct = blockIdx.x;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int hi = p.H >> i, wi = p.W >> i, ci = p.c[i];
        const int tile_lo = (ct * PC_COLS) >> i, tile_hi = min(wi, ((ct + 1) * PC_COLS) >> i);
        const int have = max(0, (tile_hi - tile_lo + 15) >> 4), S = i == 0 ? S0 : (i == 1 ? S1 : S2);
        const int rgi = RG >> i, r_begin = rg * rgi, rows = max(0, min(hi, r_begin + rgi) - r_begin);
        const float* rs = i == 0 ? rowseg0 : (i == 1 ? rowseg1 : rowseg2);
        for (int e = tid; e < rows * ci; e += nthreads) {
            const int rl = e / ci, c = e - rl * ci;
            float a = 0.f;
            for (int q = 0; q < have; ++q) a += rs[((size_t)rl * S + q) * (NT * 8) + c];
            p.rowpart[i][(((size_t)b * hi + r_begin + rl) * nct + ct) * ci + c] = a;
        }
    }
}

inline int pyr_nt(int c) {
    const int n = (c + 7) / 8;
    return n <= 2 ? 2 : n <= 3 ? 3 : n <= 4 ? 4 : n <= 6 ? 6 : 8;
}

// Tile width (multiple of 4) and the shared-memory plan; returns the total bytes, 0 if the shape does not fit.
size_t pyramid_plan(int W, int dim, const int c[3], PyramidParams* p) {
    const int nt = pyr_nt(c[0] > c[1] ? (c[0] > c[2] ? c[0] : c[2]) : (c[1] > c[2] ? c[1] : c[2]));
    const int KC = (dim + 15) / 16, xpitch = dim * 2 + 16;
    const int Wp = ((W + 3) / 4) * 4;
    // the x tile gets as much as leaves the block under 112 KB (two blocks per SM), at most 44 KB
    const int budgets[5] = {44 * 1024, 32 * 1024, 24 * 1024, 16 * 1024, 8 * 1024};
    for (int bi = 0; bi < 5; ++bi) {
        int maxTW = ((budgets[bi] / (4 * xpitch)) / 4) * 4;
        if (maxTW < 4) continue;
        const int ncol = (Wp + maxTW - 1) / maxTW;
        const int TW = (((Wp + ncol - 1) / ncol + 3) / 4) * 4;
        size_t o = (size_t)4 * TW * xpitch;
        const size_t off_p1 = o; o += (size_t)2 * (TW / 2) * xpitch;
        const size_t off_p2 = o; o += (size_t)(TW / 4) * xpitch;
        const size_t off_B = o; o += (size_t)3 * KC * nt * 32 * 8;
        const size_t off_bias = o; o += (size_t)3 * nt * 8 * 4;
        o = (o + 15) & ~size_t(15);
        const size_t off_out = o;
        o += ((size_t)4 * TW * c[0] + (size_t)2 * (TW / 2) * c[1] + (size_t)(TW / 4) * c[2]) * 2 + 16;
        o = (o + 15) & ~size_t(15);
        const size_t off_colacc = o; o += ((size_t)TW * c[0] + (size_t)(TW / 2) * c[1] + (size_t)(TW / 4) * c[2]) * 4;
        const size_t off_part = o; o += 768 * 4;
        if (o > 112 * 1024) continue;
        if (p) {
            p->TW = TW; p->KC = KC; p->xpitch = xpitch;
            p->vpp_magic = (unsigned)((0x100000000ull + (unsigned)(dim / 8) - 1) / (unsigned)(dim / 8));
            p->off_p1 = (int)off_p1; p->off_p2 = (int)off_p2; p->off_B = (int)off_B; p->off_bias = (int)off_bias; p->off_out = (int)off_out;
            p->off_colacc = (int)off_colacc; p->off_part = (int)off_part;
        }
        return o;
    }
    return 0;
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" int kad_pyramid_project_supported(int dim, int c0, int c1, int c2, int dtype, int H, int W) {
    if (!(dtype == KAD_F16 || dtype == KAD_BF16)) return 0;
    if (dim < 8 || dim % 8 != 0 || dim > 512 || H < 4 || W < 4) return 0;
    if (c0 < 1 || c1 < 1 || c2 < 1 || c0 > 64 || c1 > 64 || c2 > 64) return 0;
    const int c[3] = {c0, c1, c2};
    return pyramid_plan(W, dim, c, nullptr) != 0;
}

// Row tiles (4 rows each) one block walks through, so that a few hundred blocks remain.
static int pyramid_row_tiles_per_block(int B, int H, int n_col_tiles) {
    const long long tiles = (long long)B * ((H + 3) / 4) * n_col_tiles;
    long long rt = tiles / 592;
    return rt < 1 ? 1 : (rt > 8 ? 8 : (int)rt);
}

// Partition and shared memory of pyramid_cols_kernel; false if the shape does not qualify (the staged kernel takes it then).
static bool pyramid_cols_plan(int B, int H, int W, int dim, const int c[3], kad::ColsPlan* q) {
    using namespace kad;
    const int nt = pyr_nt(c[0] > c[1] ? (c[0] > c[2] ? c[0] : c[2]) : (c[1] > c[2] ? c[1] : c[2]));
    const int KC = (dim + 15) / 16;
    const int Wt = W < PC_COLS ? W : PC_COLS;
    ColsPlan r{};
    r.nct = (W + PC_COLS - 1) / PC_COLS;
    r.S[0] = (Wt + 15) / 16; r.S[1] = ((Wt >> 1) + 15) / 16; r.S[2] = ((Wt >> 2) + 15) / 16;
    if (r.S[1] < 1 || r.S[2] < 1) return false;
    r.warps = r.S[0] + r.S[1] + r.S[2];
    r.RT = pyramid_row_tiles_per_block(B, H, r.nct);
    if (nt >= 6) {              // wide outputs: one block per SM (registers), 37 KB of weight fragments to stage per block: about three rounds of blocks
        const long long tiles = (long long)B * ((H + 3) / 4) * r.nct;
        long long rt = (tiles + 443) / 444;
        r.RT = rt < 1 ? 1 : (rt > 8 ? 8 : (int)rt);
    }
    r.nrg = ((H + 3) / 4 + r.RT - 1) / r.RT;
    const int RG = 4 * r.RT;
    r.smem = (size_t)3 * KC * nt * 32 * 8 + (size_t)3 * nt * 8 * 4 +
             ((size_t)RG * r.S[0] + (size_t)(RG >> 1) * r.S[1] + (size_t)(RG >> 2) * r.S[2]) * nt * 8 * 4;
    if (r.smem > 100 * 1024 || r.nrg > 65535) return false;
    if (q) *q = r;
    return true;
}

extern "C" int kad_pyramid_partial_dims(int B, int H, int W, int dim, int c0, int c1, int c2, int dtype, int* n_col_tiles, int* n_row_groups) {
    KAD_CHECK_ARG(n_col_tiles && n_row_groups, "kad_pyramid_partial_dims: null pointer");
    if (!kad_pyramid_project_supported(dim, c0, c1, c2, dtype, H, W))
        return fail(KAD_ERR_UNSUPPORTED, "kad_pyramid_partial_dims: shape not supported by kad_pyramid_project");
    const int c[3] = {c0, c1, c2};
    ColsPlan q{};
    if (pyramid_cols_plan(B, H, W, dim, c, &q)) {          // the kernel kad_pyramid_project runs for this shape
        *n_col_tiles = q.nct; *n_row_groups = q.nrg;
        return KAD_OK;
    }
    PyramidParams p{};
    pyramid_plan(W, dim, c, &p);
    *n_col_tiles = (W + p.TW - 1) / p.TW;
    const int rt = pyramid_row_tiles_per_block(B, H, *n_col_tiles);
    *n_row_groups = ((H + 3) / 4 + rt - 1) / rt;
    return KAD_OK;
}

namespace kad {
namespace {
int launch_pyramid(PyramidParams& p, int dtype, cudaStream_t st) {
    const int* c = p.c;
    const size_t smem = pyramid_plan(p.W, p.dim, c, &p);
    const int nt = pyr_nt(c[0] > c[1] ? (c[0] > c[2] ? c[0] : c[2]) : (c[1] > c[2] ? c[1] : c[2]));
    ColsPlan q{};
    if (!p.counters && pyramid_cols_plan(p.B, p.H, p.W, p.dim, c, &q)) {      // (the tail variant stays with the staged kernel)
        dim3 grid(q.nct, q.nrg, p.B);
#define KAD_PYC(TT, N)                                                                                                \
    {                                                                                                                 \
        auto kern = pyramid_cols_kernel<TT, N>;                                                                       \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)q.smem);         \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "pyramid smem attribute: %s", cudaGetErrorString(e));         \
        launch_pdl(kern, grid, 32 * q.warps, q.smem, st, p, q.S[0], q.S[1], q.S[2], 4 * q.RT, q.nct, q.nrg);          \
    }
#define KAD_PYC_NT(TT)                                                                                                \
    switch (nt) { case 2: KAD_PYC(TT, 2) break; case 3: KAD_PYC(TT, 3) break; case 4: KAD_PYC(TT, 4) break;          \
                  case 6: KAD_PYC(TT, 6) break; default: KAD_PYC(TT, 8) break; }
        if (dtype == KAD_F16) { KAD_PYC_NT(__half) } else { KAD_PYC_NT(__nv_bfloat16) }
#undef KAD_PYC_NT
#undef KAD_PYC
        KAD_CHECK_LAUNCH("pyramid_cols_kernel");
        return KAD_OK;
    }
    const int nct = (p.W + p.TW - 1) / p.TW;
    p.RT = pyramid_row_tiles_per_block(p.B, p.H, nct);
    dim3 grid(nct, ((p.H + 3) / 4 + p.RT - 1) / p.RT, p.B);
    KAD_CHECK_ARG(grid.y <= 65535, "kad_pyramid_project: image too tall");
#define KAD_PYR(TT, N)                                                                                                \
    {                                                                                                                 \
        auto kern = pyramid_project_kernel<TT, N>;                                                                    \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "pyramid smem attribute: %s", cudaGetErrorString(e));         \
        kern<<<grid, MMA_THREADS, smem, st>>>(p);                                                                     \
    }
#define KAD_PYR_NT(TT)                                                                                                \
    switch (nt) { case 2: KAD_PYR(TT, 2) break; case 3: KAD_PYR(TT, 3) break; case 4: KAD_PYR(TT, 4) break;          \
                  case 6: KAD_PYR(TT, 6) break; default: KAD_PYR(TT, 8) break; }
    if (dtype == KAD_F16) { KAD_PYR_NT(__half) } else { KAD_PYR_NT(__nv_bfloat16) }
#undef KAD_PYR_NT
#undef KAD_PYR
    KAD_CHECK_LAUNCH("pyramid_project_kernel");
    return KAD_OK;
}
}  // namespace
}  // namespace kad

extern "C" int kad_pyramid_project(const void* x, const float* const* w, const float* const* bias, void* const* t,
                                   int B, int H, int W, int dim, const int* c, int dtype,
                                   float* const* rowpart, float* const* colpart, void* stream) {
    KAD_CHECK_ARG(x && w && bias && t && c, "kad_pyramid_project: null pointer");
    KAD_CHECK_ARG(B > 0 && B <= 65535, "kad_pyramid_project: bad batch %d", B);
    KAD_CHECK_ARG((rowpart == nullptr) == (colpart == nullptr), "kad_pyramid_project: rowpart and colpart go together");
    if (!kad_pyramid_project_supported(dim, c[0], c[1], c[2], dtype, H, W))
        return fail(KAD_ERR_UNSUPPORTED, "kad_pyramid_project: needs f16/bf16, dim %% 8 == 0, widths <= 64, H, W >= 4 (got dim=%d c=%d,%d,%d H=%d W=%d dtype=%d)",
                    dim, c[0], c[1], c[2], H, W, dtype);
    PyramidParams p{};
    p.x = x; p.B = B; p.H = H; p.W = W; p.dim = dim;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(w[i] && t[i], "kad_pyramid_project: null pointer for branch %d", i);
        KAD_CHECK_ARG((uintptr_t)t[i] % 4 == 0, "kad_pyramid_project: t[%d] must be 4-byte aligned", i);
        p.w[i] = w[i]; p.b[i] = bias[i]; p.t[i] = t[i]; p.c[i] = c[i];
        if (rowpart) {
            KAD_CHECK_ARG(rowpart[i] && colpart[i], "kad_pyramid_project: null partial-sum pointer for branch %d", i);
            p.rowpart[i] = rowpart[i]; p.colpart[i] = colpart[i];
        }
    }
    KAD_CHECK_ARG((uintptr_t)x % 16 == 0, "kad_pyramid_project: x must be 16-byte aligned");
    return launch_pyramid(p, dtype, (cudaStream_t)stream);
}

extern "C" int kad_pyramid_lcsa_supported(int dim, int c0, int c1, int c2, int dtype, int H, int W) {
    if (!kad_pyramid_project_supported(dim, c0, c1, c2, dtype, H, W)) return 0;
    const int c[3] = {c0, c1, c2};
    PyramidParams pp{};
    const size_t smem = pyramid_plan(W, dim, c, &pp);
    // the partial sums are laid out for the kernel kad_pyramid_project runs; the tail variant runs the staged kernel, so the
    // two partitions have to be the same one (the row groups follow from the column tiles)
    ColsPlan q{};
    if (pyramid_cols_plan(1, H, W, dim, c, &q) && q.nct != (W + pp.TW - 1) / pp.TW) return 0;
    size_t need = (size_t)W * c0 * 4;                        // the widest column-sum table (branch 0)
    if ((size_t)(W >> 1) * c1 * 4 > need) need = (size_t)(W >> 1) * c1 * 4;
    if ((size_t)(W >> 2) * c2 * 4 > need) need = (size_t)(W >> 2) * c2 * 4;
    return need <= smem ? 1 : 0;
}

extern "C" int kad_pyramid_project_lcsa(const KadPyramidArgs* a, void* stream) {
    KAD_CHECK_ARG(a && a->x && a->counters, "kad_pyramid_project_lcsa: null pointer");
    KAD_CHECK_ARG(a->B > 0 && a->B <= 65535, "kad_pyramid_project_lcsa: bad batch %d", a->B);
    if (!kad_pyramid_lcsa_supported(a->dim, a->c[0], a->c[1], a->c[2], a->dtype, a->H, a->W))
        return fail(KAD_ERR_UNSUPPORTED, "kad_pyramid_project_lcsa: shape not supported (dim=%d c=%d,%d,%d H=%d W=%d dtype=%d)",
                    a->dim, a->c[0], a->c[1], a->c[2], a->H, a->W, a->dtype);
    PyramidParams p{};
    p.x = a->x; p.B = a->B; p.H = a->H; p.W = a->W; p.dim = a->dim; p.counters = a->counters;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(a->w[i] && a->t[i] && a->rowpart[i] && a->colpart[i] && a->lcsa_w1[i] && a->lcsa_b1[i] && a->lcsa_bn_scale[i] && a->lcsa_bn_shift[i] &&
                      a->lcsa_rowmean[i] && a->lcsa_A[i] && a->lcsa_Sm[i], "kad_pyramid_project_lcsa: null pointer for branch %d", i);
        KAD_CHECK_ARG((uintptr_t)a->t[i] % 4 == 0, "kad_pyramid_project_lcsa: t[%d] must be 4-byte aligned", i);
        p.w[i] = a->w[i]; p.b[i] = a->bias[i]; p.t[i] = a->t[i]; p.c[i] = a->c[i];
        p.rowpart[i] = a->rowpart[i]; p.colpart[i] = a->colpart[i];
        p.lw1[i] = a->lcsa_w1[i]; p.lb1[i] = a->lcsa_b1[i]; p.lbn_m[i] = a->lcsa_bn_scale[i]; p.lbn_a[i] = a->lcsa_bn_shift[i];
        p.l_rowmean[i] = a->lcsa_rowmean[i]; p.l_A[i] = a->lcsa_A[i]; p.l_Sm[i] = a->lcsa_Sm[i];
    }
    KAD_CHECK_ARG((uintptr_t)a->x % 16 == 0, "kad_pyramid_project_lcsa: x must be 16-byte aligned");
    return launch_pyramid(p, a->dtype, (cudaStream_t)stream);
}
