// 3x3 convolution (padding 1, stride 1 or 2) + bias + activation as a TMA-fed tcgen05 implicit GEMM for sm_100a.
//
//   y[b][yo][xo][n] = act( sum_{ky,kx,c} x[b][s*yo+ky-1][s*xo+kx-1][c] * w[n][ky*3+kx][c] + bias[n] )
//
// NHWC activations make every filter tap of an output tile a plain 4-D box of the input: the tile is a th x tw
// rectangle of output pixels of one image (th*tw <= 128, chosen per shape so that the tiles cover the map with the
// least padding), and the A operand of tap (ky,kx) and channel chunk c0 is the box [th][tw][64 channels] whose corner
// is shifted by the tap. TMA writes it in the canonical 128-byte-swizzled K-major layout (one pixel = one 128-byte
// row) and fills rows and channels outside the tensor with zeros, which is the convolution's zero padding and the
// K padding at once; no im2col buffer exists anywhere. Stride 2 uses four tensor maps, one per (row, column) parity
// of the input, so that the pixels a tap needs are again a dense box.
// The weights [Cout][9][Cin] are a 3-D tensor map (channel, tap, output channel); a stage is one (tap, chunk) pair.
// One persistent CTA per SM: warps 0-7 epilogue (TMEM -> bias/activation -> NHWC store, also into a channel slice of
// a wider tensor), warp 8 issues the MMAs, warp 9 the TMA loads; the accumulator is double buffered in TMEM.
#include "kad_common.cuh"
#include "kad_sm100.cuh"

namespace kad {
namespace {
using namespace sm100;

constexpr int CMAX_STAGES = 10;
constexpr int C_A_BYTES = 128 * 128;
constexpr int C_THREADS = 320;
constexpr int C_EPI_WARPS = 8, C_WARP_MMA = 8;
constexpr int C_ACC_COLS = 256;

struct ConvMaps {
    CUtensorMap a[4];      // stride 1: a[0]; stride 2: a[py * 2 + px], the input pixels of row parity py and column parity px
    CUtensorMap b;
};

struct ConvParams {
    const float* bias; void* y; int* status;
    int B, Ho, Wo, Cin, N, ldy, act, fmt, stride;
    int th, tw, tiles_y, tiles_x;
    int nt, n_tiles, chunks;
    long long m_tiles;
    int b_stage_bytes, stages;
};

struct ConvBars {
    uint64_t full[CMAX_STAGES], empty[CMAX_STAGES];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void creport(int* status, int code, int detail) {
    if (atomicCAS(status, 0, code) == 0) { status[1] = detail; status[2] = blockIdx.x; }
}

template <typename T>
__global__ void __launch_bounds__(C_THREADS, 1)
conv3x3_tc_kernel(const __grid_constant__ ConvMaps maps, const ConvParams p) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* sa = smem;
    const int STAGES = p.stages;
    unsigned char* sb = smem + STAGES * C_A_BYTES;
    ConvBars* bars = reinterpret_cast<ConvBars*>(sb + STAGES * p.b_stage_bytes);
    volatile int* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long ntiles = p.m_tiles * p.n_tiles;
    const int ksteps = 9 * p.chunks;

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 1); mbar_init(&bars->acc_empty[i], C_EPI_WARPS * 32); }
        bars->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == C_WARP_MMA) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
    float* sbias = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + ((sizeof(ConvBars) + 15) & ~size_t(15)));
    for (int i = tid; i < p.n_tiles * p.nt; i += C_THREADS) sbias[i] = (p.bias && i < p.N) ? p.bias[i] : 0.f;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    const int tiles_per_image = p.tiles_y * p.tiles_x;

    if (warp < C_EPI_WARPS) {
        const int quad = warp & 3, half = warp >> 2;
        const int r = quad * 32 + lane;                    // accumulator row = pixel (r / tw, r % tw) of the tile
        const int ty = r / p.tw, tx = r - ty * p.tw;
        int it = 0;
        for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_full[buf], (it >> 1) & 1, abort_flag)) { creport(p.status, 1, it); break; }
            tc_fence_after();
            const long long mt = tile / p.n_tiles;
            const int n0 = (int)(tile - mt * p.n_tiles) * p.nt;
            const int img = (int)(mt / tiles_per_image);
            const int rem = (int)(mt - (long long)img * tiles_per_image);
            const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
            const int yo = tyi * p.th + ty, xo = txi * p.tw + tx;
            const bool live = ty < p.th && yo < p.Ho && xo < p.Wo;
            const long long row = ((long long)img * p.Ho + yo) * p.Wo + xo;
            const int nchunks = (p.nt + 31) / 32;
            for (int ch = half; ch < nchunks; ch += 2) {
                const int c0 = ch * 32;
                const int nc = min(32, p.nt - c0);
                uint32_t v[32];
                const uint32_t taddr = tmem_base + (uint32_t)(buf * C_ACC_COLS + c0) + ((uint32_t)(quad * 32) << 16);
                if (nc > 16) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
                tmem_ld_wait();
                if (live) {
                    T* dst = reinterpret_cast<T*>(p.y) + row * p.ldy + n0 + c0;
                    const float4* b4 = reinterpret_cast<const float4*>(sbias + n0 + c0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int n = n0 + c0 + 8 * j;
                        if (8 * j < nc && n < p.N) {      // N % 8 == 0: a group of 8 is all in or all out
                            const float4 ba = b4[2 * j], bb = b4[2 * j + 1];
                            float a[8] = {__uint_as_float(v[8 * j + 0]) + ba.x, __uint_as_float(v[8 * j + 1]) + ba.y,
                                          __uint_as_float(v[8 * j + 2]) + ba.z, __uint_as_float(v[8 * j + 3]) + ba.w,
                                          __uint_as_float(v[8 * j + 4]) + bb.x, __uint_as_float(v[8 * j + 5]) + bb.y,
                                          __uint_as_float(v[8 * j + 6]) + bb.z, __uint_as_float(v[8 * j + 7]) + bb.w};
                            uint4 w;
                            T* h = reinterpret_cast<T*>(&w);
                            if (p.act == KAD_ACT_SILU) {
                                // x * sigmoid(x) = x * (0.5 * tanh(x / 2) + 0.5): one special-function instruction per element
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    float th;
                                    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * a[e]));
                                    h[e] = from_f<T>(a[e] * fmaf(0.5f, th, 0.5f));
                                }
                            } else if (p.act == KAD_ACT_RELU) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = from_f<T>(fmaxf(a[e], 0.f));
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = from_f<T>(a[e]);
                            }
                            *reinterpret_cast<uint4*>(dst + 8 * j) = w;
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[buf]);
        }
    } else if (warp == C_WARP_MMA) {
        const uint32_t idesc = instr_desc_f16(p.fmt, p.nt);
        const uint32_t a_base = smem_u32(sa), b_base = smem_u32(sb);
        const int last_nk = (p.Cin - (p.chunks - 1) * 64 + 15) / 16;      // 16-wide K steps of a tap's last channel chunk
        int it = 0;
        int slot = 0; uint32_t phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) { creport(p.status, 2, it); break; }
            tc_fence_after();
            const uint32_t tacc = tmem_base + (uint32_t)(buf * C_ACC_COLS);
            int ch = 0;
            for (int s = 0; s < ksteps; ++s) {
                if (!mbar_wait(&bars->full[slot], phase, abort_flag)) { creport(p.status, 3, s); ok = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t aaddr = a_base + slot * C_A_BYTES, baddr = b_base + slot * p.b_stage_bytes;
                    const int nk = (ch == p.chunks - 1) ? last_nk : 4;
                    for (int k = 0; k < nk; ++k)
                        umma_f16(tacc, smem_desc_sw128(aaddr + k * 32), smem_desc_sw128(baddr + k * 32), idesc, (s | k) ? 1u : 0u);
                    umma_commit(&bars->empty[slot]);
                    if (s == ksteps - 1) umma_commit(&bars->acc_full[buf]);
                }
                __syncwarp();
                if (++ch == p.chunks) ch = 0;
                if (++slot == STAGES) { slot = 0; phase ^= 1u; }
            }
        }
    } else {
        if (lane == 0) {
            for (int i = 0; i < (p.stride == 2 ? 4 : 1); ++i) tma_prefetch_desc(&maps.a[i]);
            tma_prefetch_desc(&maps.b);
            long long is = 0;
            int slot = 0; uint32_t phase = 0;
            bool ok = true;
            const uint32_t tx_bytes = (uint32_t)(p.th * p.tw * 128 + p.nt * 128);
            for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const long long mt = tile / p.n_tiles;
                const int n0 = (int)(tile - mt * p.n_tiles) * p.nt;
                const int img = (int)(mt / tiles_per_image);
                const int rem = (int)(mt - (long long)img * tiles_per_image);
                const int tyi = rem / p.tiles_x, txi = rem - tyi * p.tiles_x;
                const int y0 = tyi * p.th, x0 = txi * p.tw;
                for (int tap = 0; tap < 9 && ok; ++tap) {
                    const int ky = tap / 3, kx = tap - ky * 3;
                    // stride 1: input pixel (y0 + ky - 1, x0 + kx - 1). stride 2: input row 2*yo + ky - 1 has parity
                    // (ky != 1) and index yo - (ky == 0) among the rows of that parity; columns alike.
                    const CUtensorMap* ma = p.stride == 2 ? &maps.a[(ky != 1) * 2 + (kx != 1)] : &maps.a[0];
                    const int cy = p.stride == 2 ? y0 - (ky == 0) : y0 + ky - 1;
                    const int cx = p.stride == 2 ? x0 - (kx == 0) : x0 + kx - 1;
                    for (int ch = 0; ch < p.chunks; ++ch, ++is) {
                        if (!mbar_wait(&bars->empty[slot], phase ^ 1u, abort_flag)) { creport(p.status, 4, tap); ok = false; break; }
                        mbar_arrive_expect_tx(&bars->full[slot], tx_bytes);
                        tma_load_4d(sa + slot * C_A_BYTES, ma, ch * 64, cx, cy, img, &bars->full[slot]);
                        tma_load_3d(sb + slot * p.b_stage_bytes, &maps.b, ch * 64, tap, n0, &bars->full[slot]);
                        if (++slot == STAGES) { slot = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok || *abort_flag) {
                // the copies already issued must land before the block may exit
                for (int i = 0; i < STAGES && i < is; ++i) {
                    long long j = is - 1 - i;
                    mbar_wait(&bars->full[j % STAGES], (uint32_t)((j / STAGES) & 1), abort_flag);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == C_WARP_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
    if (tid == 0 && *abort_flag) creport(p.status, 9, 0);
}

}  // namespace
}  // namespace kad

using namespace kad;
using namespace kad::sm100;

extern "C" int kad_conv3x3_tc_supported(int Cin, int Cout, int stride, int dtype) {
    return (dtype == KAD_F16 || dtype == KAD_BF16) && Cin >= 8 && Cin % 8 == 0 && Cout >= 8 && Cout % 8 == 0 && (stride == 1 || stride == 2);
}

extern "C" int kad_conv3x3_bias_act(const void* x, const void* w, const float* bias, void* y,
                                    int B, int H, int W, int Cin, int Cout, int stride, int ldx, int ldy, int act, int dtype,
                                    int* status, void* stream) {
    KAD_CHECK_ARG(x && w && y && status, "kad_conv3x3_bias_act: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0, "kad_conv3x3_bias_act: bad shape [%d,%d,%d]", B, H, W);
    if (!kad_conv3x3_tc_supported(Cin, Cout, stride, dtype))
        return fail(KAD_ERR_UNSUPPORTED, "kad_conv3x3_bias_act: needs f16/bf16, Cin %% 8 == 0, Cout %% 8 == 0, stride 1 or 2 (Cin=%d Cout=%d stride=%d dtype=%d)",
                    Cin, Cout, stride, dtype);
    KAD_CHECK_ARG(stride == 1 || (H >= 2 && W >= 2), "kad_conv3x3_bias_act: stride 2 needs H, W >= 2");
    KAD_CHECK_ARG(ldx >= Cin && ldx % 8 == 0 && ldy >= Cout && ldy % 8 == 0, "kad_conv3x3_bias_act: ldx/ldy must be >= Cin/Cout and multiples of 8");
    KAD_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0), "kad_conv3x3_bias_act: pointers must be 16-byte aligned");
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(KAD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");

    ConvParams p{};
    p.bias = bias; p.y = y; p.status = status;
    p.B = B; p.Cin = Cin; p.N = Cout; p.ldy = ldy; p.act = act; p.stride = stride;
    p.Ho = (H - 1) / stride + 1; p.Wo = (W - 1) / stride + 1;          // kernel 3, padding 1
    p.fmt = dtype == KAD_BF16 ? 1 : 0;
    // output tile th x tw (<= 128 pixels) that covers the map with the fewest tiles; ties go to the wider tile
    {
        long long best = -1;
        for (int th = 1; th <= 128 && th <= p.Ho; ++th) {
            int tw = 128 / th; if (tw > p.Wo) tw = p.Wo;
            long long t = (long long)((p.Ho + th - 1) / th) * ((p.Wo + tw - 1) / tw);
            if (best < 0 || t < best) { best = t; p.th = th; p.tw = tw; }
        }
    }
    p.tiles_y = (p.Ho + p.th - 1) / p.th; p.tiles_x = (p.Wo + p.tw - 1) / p.tw;
    p.m_tiles = (long long)B * p.tiles_y * p.tiles_x;
    p.n_tiles = (Cout + 255) / 256;
    p.nt = ((Cout + p.n_tiles - 1) / p.n_tiles + 15) & ~15;
    p.chunks = (Cin + 63) / 64;
    p.b_stage_bytes = p.nt * 128;

    ConvMaps maps;
    CUtensorMapDataType dt = dtype == KAD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    for (int q = 0; q < (stride == 2 ? 4 : 1); ++q) {
        const int py = q >> 1, px = q & 1;
        // the pixels of row parity py and column parity px (stride 2), or all pixels (stride 1)
        const int Hq = stride == 2 ? (H - py + 1) / 2 : H, Wq = stride == 2 ? (W - px + 1) / 2 : W;
        const char* base = reinterpret_cast<const char*>(x) + (stride == 2 ? ((size_t)py * W + px) * ldx * 2 : 0);
        cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)Wq, (cuuint64_t)Hq, (cuuint64_t)B};
        cuuint64_t strides[3] = {(cuuint64_t)stride * ldx * 2, (cuuint64_t)stride * W * ldx * 2, (cuuint64_t)H * W * ldx * 2};
        cuuint32_t box[4] = {64, (cuuint32_t)p.tw, (cuuint32_t)p.th, 1};
        CUresult r = enc(&maps.a[q], dt, 4, const_cast<char*>(base), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for x failed (CUresult %d)", (int)r);
    }
    {
        cuuint64_t dims[3] = {(cuuint64_t)Cin, 9, (cuuint64_t)Cout};
        cuuint64_t strides[2] = {(cuuint64_t)Cin * 2, (cuuint64_t)9 * Cin * 2};
        cuuint32_t box[3] = {64, 1, (cuuint32_t)p.nt};
        CUresult r = enc(&maps.b, dt, 3, const_cast<void*>(w), dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for w failed (CUresult %d)", (int)r);
    }
    const size_t fixed = sizeof(ConvBars) + (size_t)p.n_tiles * p.nt * 4 + 1024 + 128;
    int stages = (int)((200 * 1024 - fixed) / (size_t)(C_A_BYTES + p.b_stage_bytes));
    stages = stages < 2 ? 2 : (stages > CMAX_STAGES ? CMAX_STAGES : stages);
    p.stages = stages;
    const size_t smem = (size_t)stages * (C_A_BYTES + p.b_stage_bytes) + fixed;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long ntiles = p.m_tiles * p.n_tiles;
    const int grid = (int)(ntiles < sms ? ntiles : sms);
    cudaError_t e;
    if (dtype == KAD_F16) {
        auto kern = conv3x3_tc_kernel<__half>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "conv3x3 smem attribute: %s", cudaGetErrorString(e));
        kern<<<grid, C_THREADS, smem, (cudaStream_t)stream>>>(maps, p);
    } else {
        auto kern = conv3x3_tc_kernel<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "conv3x3 smem attribute: %s", cudaGetErrorString(e));
        kern<<<grid, C_THREADS, smem, (cudaStream_t)stream>>>(maps, p);
    }
    KAD_CHECK_LAUNCH("conv3x3_tc_kernel");
    return KAD_OK;
}
