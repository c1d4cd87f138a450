// First layer of the detector on raw images: uint8 [B,Cin,H,W] planes -> 3x3 convolution, stride 2, padding 1 ->
// * scale (the 1/255 normalisation) + bias -> SiLU -> NHWC fp16/bf16, in one kernel.
//
// The layer is memory-bound (3 bytes in, 2*Cout bytes out per output pixel, 27*Cout MACs), but on CUDA cores the MACs
// and the SiLU would take longer than the traffic. So the contraction runs on the warp-level tensor-core instruction
// (mma.sync m16n8k16): K = Cin*9 <= 48 padded to 16-chunks, pixel values enter as exact fp16 integers 0..255 and the
// 1/255 is applied to the fp32 accumulator; SiLU uses the hardware exponential and reciprocal. A block owns 8 x 32 output pixels;
// its (17 x 65 x Cin)-byte input patch goes through shared memory, and each warp's 32 output pixels leave as one
// contiguous run of 16-byte vectors.
#include "kad_mma.cuh"

namespace kad {
namespace {

constexpr int STEM_THREADS = 256;
constexpr int ST_ROWS = 8, ST_COLS = 32;                  // output pixels per block
constexpr int ST_IN_ROWS = 2 * ST_ROWS + 1, ST_IN_COLS = 2 * ST_COLS + 1;
constexpr int ST_PITCH = 72;                              // bytes per staged input row (18 words: the row may start 3 bytes into the first)
constexpr int ST_MAX_CIN = 4, ST_MAX_NT = 8;

template <typename T> __device__ __forceinline__ uint32_t st_pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t st_pack2<__half>(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
template <> __device__ __forceinline__ uint32_t st_pack2<__nv_bfloat16>(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }

template <typename T> __device__ __forceinline__ void st_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b);
template <> __device__ __forceinline__ void st_mma<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}
template <> __device__ __forceinline__ void st_mma<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}

__device__ __forceinline__ float fast_silu(float v) { return silu_fast(v); }

// K index of the contraction: k = ci*9 + ky*3 + kx (the flattening of an [Cout][Cin][3][3] weight). Lane t of a 16-chunk
// owns k = chunk*16 + {2t, 2t+1, 2t+8, 2t+9} (the operand layout of mma.sync, no permutation needed here).
template <typename T, int NT, int KC, bool WORDS>
__global__ void __launch_bounds__(STEM_THREADS, NT <= 5 ? 4 : 2)
stem_conv_kernel(const unsigned char* __restrict__ img, const float* __restrict__ w, const float* __restrict__ bias, T* __restrict__ y,
                 int Cin, int H, int W, int OH, int OW, int Cout, float scale, int act, int tiles_per_block) {
    // WORDS (W % 4 == 0, image 4-byte aligned): the patch is staged as aligned 4-byte words by asynchronous copies, the patch of
    // the next row tile while the current one is computed; a row of the patch then starts 3 bytes into its first word.
    __shared__ __align__(16) unsigned char patches[2][ST_MAX_CIN * ST_IN_ROWS * ST_PITCH];
    __shared__ uint2 Bs[KC * NT * 32];
    __shared__ float bs[NT * 8];
    __shared__ int koff[KC * 16];                          // byte offset of k inside the patch, relative to the pixel's corner; -1: padding
    __shared__ __align__(16) unsigned char tiles[STEM_THREADS / 32][32 * NT * 8 * 2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, ox0 = blockIdx.x * ST_COLS;
    const int ix0 = 2 * ox0 - 1;
    const int K = Cin * 9;
    constexpr int SHIFT = WORDS ? 3 : 0;                    // patch column of input column ix0
    const int ty0 = blockIdx.y * tiles_per_block, nty = (OH + ST_ROWS - 1) / ST_ROWS;
    const int ntiles = min(tiles_per_block, nty - ty0);

    const unsigned char* ib = img + (size_t)b * Cin * H * W;
    // input patch of row tile ty (zero outside the image)
    auto stage_patch = [&](int ty, unsigned char* patch) {
        const int iy0 = 2 * ty * ST_ROWS - 1;
        if (WORDS) {
            constexpr int WPR = ST_PITCH / 4;
            const int xa0 = ix0 - 3;                            // a multiple of 4
            for (int e = tid; e < Cin * ST_IN_ROWS * WPR; e += STEM_THREADS) {
                const int wd = e % WPR, r = (e / WPR) % ST_IN_ROWS, ci = e / (WPR * ST_IN_ROWS);
                const int yy = iy0 + r, xx = xa0 + 4 * wd;
                unsigned char* dst = patch + (ci * ST_IN_ROWS + r) * ST_PITCH + 4 * wd;
                if (yy >= 0 && yy < H && xx >= 0 && xx < W) cp_async4(dst, ib + ((size_t)ci * H + yy) * W + xx);
                else *reinterpret_cast<uint32_t*>(dst) = 0u;
            }
        } else {
            for (int e = tid; e < Cin * ST_IN_ROWS * ST_PITCH; e += STEM_THREADS) {
                const int c = e % ST_PITCH, r = (e / ST_PITCH) % ST_IN_ROWS, ci = e / (ST_PITCH * ST_IN_ROWS);
                const int yy = iy0 + r, xx = ix0 + c;
                patch[e] = (c < ST_IN_COLS && yy >= 0 && yy < H && xx >= 0 && xx < W) ? ib[((size_t)ci * H + yy) * W + xx] : (unsigned char)0;
            }
        }
    };
    if (ntiles > 0) stage_patch(ty0, patches[0]);
    cp_async_commit();
    for (int e = tid; e < KC * NT * 32; e += STEM_THREADS) {
        const int l = e & 31, nt = (e >> 5) % NT, kc = (e >> 5) / NT;
        const int n = nt * 8 + (l >> 2), k0 = kc * 16 + 2 * (l & 3);
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + (j & 1) + (j >> 1) * 8;
            v[j] = (n < Cout && k < K) ? w[(size_t)n * K + k] : 0.f;
        }
        Bs[e] = make_uint2(st_pack2<T>(v[0], v[1]), st_pack2<T>(v[2], v[3]));
    }
    for (int e = tid; e < NT * 8; e += STEM_THREADS) bs[e] = (e < Cout && bias) ? bias[e] : 0.f;
    for (int k = tid; k < KC * 16; k += STEM_THREADS) {
        const int ci = k / 9, r = (k % 9) / 3, c = k % 3;
        koff[k] = k < K ? (ci * ST_IN_ROWS + r) * ST_PITCH + c + SHIFT : -1;
    }

    for (int kt = 0; kt < ntiles; ++kt) {
    const unsigned char* patch = patches[kt & 1];
    const int oy0 = (ty0 + kt) * ST_ROWS;
    if (kt + 1 < ntiles) stage_patch(ty0 + kt + 1, patches[(kt + 1) & 1]);      // in flight while this tile is computed
    cp_async_commit();
    cp_async_wait_but_one();                                                    // this tile's patch has landed
    __syncthreads();

    // this warp: output row oy0 + warp, 32 pixels = two 16-row tiles; lane rows g and g+8
    float acc[2][NT][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
#pragma unroll
    for (int kc = 0; kc < KC; ++kc) {
        int ko[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) ko[j] = koff[kc * 16 + 2 * t + (j & 1) + (j >> 1) * 8];
        uint32_t a[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int px = mt * 16 + g + 8 * h;                       // output column inside the tile
                const int corner = (2 * warp) * ST_PITCH + 2 * px;         // patch offset of input (2*oy-1, 2*ox-1) in plane 0
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = ko[j] >= 0 ? (float)patch[corner + ko[j]] : 0.f;
                a[mt][h] = st_pack2<T>(v[0], v[1]);
                a[mt][2 + h] = st_pack2<T>(v[2], v[3]);
            }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint2 bf = Bs[(kc * NT + nt) * 32 + lane];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) st_mma<T>(acc[mt][nt], a[mt][0], a[mt][1], a[mt][2], a[mt][3], bf);
        }
    }

    // epilogue through the warp's tile: [32 pixels][Cout]
    const int oy = oy0 + warp;
    unsigned char* tile = tiles[warp];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int px = mt * 16 + g + 8 * h;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int co = nt * 8 + 2 * t;
                if (co >= Cout) continue;
                float v0 = fmaf(acc[mt][nt][2 * h], scale, bs[co]), v1 = fmaf(acc[mt][nt][2 * h + 1], scale, bs[co + 1]);
                if (act == KAD_ACT_SILU) { v0 = fast_silu(v0); v1 = fast_silu(v1); }
                else if (act == KAD_ACT_RELU) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
                *reinterpret_cast<uint32_t*>(tile + ((size_t)px * Cout + co) * 2) = st_pack2<T>(v0, v1);
            }
        }
    __syncwarp();
    if (oy < OH) {
        const int npx = min(ST_COLS, OW - ox0);
        if (npx > 0) {
            const int nb = npx * Cout * 2;                                  // a multiple of 16: Cout % 8 == 0
            uint4* dst = reinterpret_cast<uint4*>(y + (((size_t)b * OH + oy) * OW + ox0) * Cout);
            const uint4* src = reinterpret_cast<const uint4*>(tile);
            for (int i = lane; i < (nb >> 4); i += 32) dst[i] = src[i];
        }
    }
    __syncthreads();                     // every warp is done with this patch (the tile after the next lands in it) and with its output tile
    }   // row tiles
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" int kad_stem_conv_supported(int Cin, int Cout, int dtype) {
    return (dtype == KAD_F16 || dtype == KAD_BF16) && Cin >= 1 && Cin <= ST_MAX_CIN && Cout >= 8 && Cout <= ST_MAX_NT * 8 && Cout % 8 == 0;
}

extern "C" int kad_stem_conv_u8(const void* img_u8, const float* w_oihw, const float* bias, void* y,
                                int B, int Cin, int H, int W, int Cout, float scale, int act, int dtype, void* stream) {
    KAD_CHECK_ARG(img_u8 && w_oihw && y, "kad_stem_conv_u8: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && B <= 65535, "kad_stem_conv_u8: bad shape");
    if (!kad_stem_conv_supported(Cin, Cout, dtype))
        return fail(KAD_ERR_UNSUPPORTED, "kad_stem_conv_u8: needs f16/bf16, Cin <= %d, Cout a multiple of 8 up to %d (got Cin=%d Cout=%d dtype=%d)",
                    ST_MAX_CIN, ST_MAX_NT * 8, Cin, Cout, dtype);
    KAD_CHECK_ARG((uintptr_t)y % 16 == 0, "kad_stem_conv_u8: y must be 16-byte aligned");
    KAD_CHECK_ARG(act == KAD_ACT_NONE || act == KAD_ACT_SILU || act == KAD_ACT_RELU, "kad_stem_conv_u8: unknown activation %d", act);
    const int OH = (H - 1) / 2 + 1, OW = (W - 1) / 2 + 1;
    // row tiles per block: the weights are staged once per block and the next patch loads during a tile, so a block takes several
    // tiles as long as a few thousand blocks remain
    const int nty = (OH + ST_ROWS - 1) / ST_ROWS, ntx = (OW + ST_COLS - 1) / ST_COLS;
    int tpb = (int)(((long long)nty * ntx * B) / 4096);
    tpb = tpb < 1 ? 1 : (tpb > 8 ? 8 : tpb);
    dim3 grid(ntx, (nty + tpb - 1) / tpb, B);
    KAD_CHECK_ARG(grid.y <= 65535, "kad_stem_conv_u8: image too tall");
    const bool words = W % 4 == 0 && (uintptr_t)img_u8 % 4 == 0 && ((size_t)H * W) % 4 == 0;
    const int nt = (Cout + 7) / 8, kc = (Cin * 9 + 15) / 16;
    cudaStream_t st = (cudaStream_t)stream;
#define KAD_STEM(TT, N, KCC)                                                                                                                          \
    { if (words) stem_conv_kernel<TT, N, KCC, true><<<grid, STEM_THREADS, 0, st>>>((const unsigned char*)img_u8, w_oihw, bias, (TT*)y, Cin, H, W, OH, OW, Cout, scale, act, tpb); \
      else stem_conv_kernel<TT, N, KCC, false><<<grid, STEM_THREADS, 0, st>>>((const unsigned char*)img_u8, w_oihw, bias, (TT*)y, Cin, H, W, OH, OW, Cout, scale, act, tpb); }
#define KAD_STEM_NT(TT, KCC)                                                                                      \
    switch (nt) {                                                                                                 \
        case 1: KAD_STEM(TT, 1, KCC) break; case 2: KAD_STEM(TT, 2, KCC) break; case 3: KAD_STEM(TT, 3, KCC) break; \
        case 4: KAD_STEM(TT, 4, KCC) break; case 5: KAD_STEM(TT, 5, KCC) break; case 6: KAD_STEM(TT, 6, KCC) break; \
        case 7: KAD_STEM(TT, 7, KCC) break; default: KAD_STEM(TT, 8, KCC) break;                               \
    }
#define KAD_STEM_KC(TT)                                                                                           \
    switch (kc) { case 1: KAD_STEM_NT(TT, 1) break; case 2: KAD_STEM_NT(TT, 2) break; default: KAD_STEM_NT(TT, 3) break; }
    if (dtype == KAD_F16) { KAD_STEM_KC(__half) } else { KAD_STEM_KC(__nv_bfloat16) }
#undef KAD_STEM_KC
#undef KAD_STEM_NT
#undef KAD_STEM
    KAD_CHECK_LAUNCH("stem_conv_kernel");
    return KAD_OK;
}
