// 1x1 convolution + bias + activation as a TMA-fed tcgen05 GEMM for sm_100a.
//
//   y[m][n] = act( sum_k x[m][k] * w[n][k] + bias[n] ),  m = pixel (NHWC rows), k = Cin, n = Cout.
//
// Both operands are K-major in global memory already (NHWC activations, [Cout][Cin] weights), so
// each pipeline stage is two plain tiled TMA loads (128 x 64 of x, Nt x 64 of w, 128-byte swizzle;
// out-of-range K and N are zero-filled by TMA). One persistent CTA per SM:
//   warps 0-7 epilogue (TMEM -> bias/activation -> NHWC store; warps w and w+4 share a TMEM lane quadrant and split
//   the columns), warp 8 MMA issuer, warp 9 TMA.
// The op is HBM-bound at the detector's shapes (K <= 512): the design goal is to keep enough bytes
// in flight, which a ring of 4 to 10 stages (as many as fit beside the weight tile) and the double-buffered accumulator do;
// the weight tile is loaded once per CTA and stays in shared memory when it fits (it is the same for every M tile).
#include "kad_common.cuh"
#include "kad_sm100.cuh"

namespace kad {
namespace {
using namespace sm100;

constexpr int GBM = 128;
constexpr int GMAX_STAGES = 10;      // ring depth is chosen per shape: as many stages as fit (narrow outputs get a deeper ring)
constexpr int G_A_BYTES = GBM * 128;
constexpr int G_THREADS = 320;
constexpr int G_EPI_WARPS = 8, G_WARP_MMA = 8;      // warp 9 issues the TMA loads
constexpr int G_ACC_COLS = 256;

struct GemmParams {
    const float* bias; void* y; int* status;
    long long M; int K, N, ldy, act, fmt;
    int nt;            // output-channel tile (multiple of 16, <= 256)
    int n_tiles, m_tiles, ksteps;
    int b_stage_bytes;
    int stages;
    int resident;      // 1: all K slices of the weight tile stay in shared memory for the whole kernel (one output-channel tile)
};

struct GemmBars {
    uint64_t full[GMAX_STAGES], empty[GMAX_STAGES];
    uint64_t acc_full[2], acc_empty[2];
    uint64_t w_full;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void greport(int* status, int code, int detail) {
    if (atomicCAS(status, 0, code) == 0) { status[1] = detail; status[2] = blockIdx.x; }
}

template <typename T>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm1x1_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* sa = smem;
    const int GSTAGES = p.stages;
    unsigned char* sb = smem + GSTAGES * G_A_BYTES;
    GemmBars* bars = reinterpret_cast<GemmBars*>(sb + (p.resident ? p.ksteps : GSTAGES) * p.b_stage_bytes);
    volatile int* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long ntiles = (long long)p.m_tiles * p.n_tiles;

    if (tid == 0) {
        for (int i = 0; i < GSTAGES; ++i) { mbar_init(&bars->full[i], 1); mbar_init(&bars->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 1); mbar_init(&bars->acc_empty[i], G_EPI_WARPS * 32); }
        mbar_init(&bars->w_full, 1);
        bars->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == G_WARP_MMA) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
    // bias of every output channel, padded with zeros to the tile grid
    float* sbias = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + ((sizeof(GemmBars) + 15) & ~size_t(15)));   // 16-byte aligned: read as float4
    for (int i = tid; i < p.n_tiles * p.nt; i += G_THREADS) sbias[i] = (p.bias && i < p.N) ? p.bias[i] : 0.f;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;
    // barriers, tensor memory and the bias are set up: with a programmatic launch that happened while the kernel before drained
    grid_dependency_wait();
    grid_dependents_go();

    if (warp < G_EPI_WARPS) {
        const int quad = warp & 3, half = warp >> 2;       // TMEM lane quadrant; which half of the column chunks
        int it = 0;
        for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_full[buf], (it >> 1) & 1, abort_flag)) { greport(p.status, 1, it); break; }
            tc_fence_after();
            const long long mt = tile / p.n_tiles;
            const int n0 = (int)(tile - mt * p.n_tiles) * p.nt;
            const long long row = mt * GBM + quad * 32 + lane;
            const bool live = row < p.M;
            const int nchunks = (p.nt + 31) / 32;
            for (int ch = half; ch < nchunks; ch += 2) {
                const int c0 = ch * 32;
                const int nc = min(32, p.nt - c0);
                uint32_t v[32];
                const uint32_t taddr = tmem_base + (uint32_t)(buf * G_ACC_COLS + c0) + ((uint32_t)(quad * 32) << 16);
                if (nc == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
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
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = from_f<T>(silu_fast(a[e]));
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
    } else if (warp == G_WARP_MMA) {
        const uint32_t idesc = instr_desc_f16(p.fmt, p.nt);
        const uint32_t a_base = smem_u32(sa), b_base = smem_u32(sb);
        int it = 0;
        int slot = 0; uint32_t phase = 0;          // ring position (wrap counters: no division in this loop)
        bool ok = true;
        if (p.resident && !mbar_wait(&bars->w_full, 0, abort_flag)) { greport(p.status, 5, 0); ok = false; }
        for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) { greport(p.status, 2, it); break; }
            tc_fence_after();
            const uint32_t tacc = tmem_base + (uint32_t)(buf * G_ACC_COLS);
            for (int s = 0; s < p.ksteps; ++s) {
                if (!mbar_wait(&bars->full[slot], phase, abort_flag)) { greport(p.status, 3, s); ok = false; break; }
                if (lane == 0) {
                    const uint32_t aaddr = a_base + slot * G_A_BYTES, baddr = b_base + (p.resident ? s : slot) * p.b_stage_bytes;
                    // K beyond the tensor extent is zero-filled in both operands, so a full stage is always safe
                    const int kleft = p.K - s * 64;
                    const int nk = kleft >= 64 ? 4 : (kleft + 15) / 16;
                    for (int k = 0; k < nk; ++k)
                        umma_f16(tacc, smem_desc_sw128(aaddr + k * 32), smem_desc_sw128(baddr + k * 32), idesc, (s | k) ? 1u : 0u);
                    umma_commit(&bars->empty[slot]);
                    if (s == p.ksteps - 1) umma_commit(&bars->acc_full[buf]);
                }
                __syncwarp();
                if (++slot == GSTAGES) { slot = 0; phase ^= 1u; }
            }
        }
    } else {
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            long long is = 0;
            int slot = 0; uint32_t phase = 0;
            bool ok = true;
            // resident weights: every K slice of the (only) output-channel tile once, on a barrier of its own; the MMA warp
            // waits for them before its first instruction, so they have landed long before the block can exit
            if (p.resident) {
                mbar_arrive_expect_tx(&bars->w_full, (uint32_t)(p.ksteps * p.nt * 128));
                for (int s = 0; s < p.ksteps; ++s) tma_load_2d(sb + s * p.b_stage_bytes, &map_b, s * 64, 0, &bars->w_full);
            }
            const uint32_t tx = (uint32_t)(G_A_BYTES + (p.resident ? 0 : p.nt * 128));
            for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const long long mt = tile / p.n_tiles;
                const int n0 = (int)(tile - mt * p.n_tiles) * p.nt;
                for (int s = 0; s < p.ksteps; ++s, ++is) {
                    if (!mbar_wait(&bars->empty[slot], phase ^ 1u, abort_flag)) { greport(p.status, 4, s); ok = false; break; }
                    mbar_arrive_expect_tx(&bars->full[slot], tx);
                    tma_load_2d(sa + slot * G_A_BYTES, &map_a, s * 64, (int)(mt * GBM), &bars->full[slot]);
                    if (!p.resident) tma_load_2d(sb + slot * p.b_stage_bytes, &map_b, s * 64, n0, &bars->full[slot]);
                    if (++slot == GSTAGES) { slot = 0; phase ^= 1u; }
                }
            }
            if (!ok || *abort_flag) {
                // the copies already issued must land before the block may exit
                for (int i = 0; i < GSTAGES && i < is; ++i) {
                    long long j = is - 1 - i;
                    mbar_wait(&bars->full[j % GSTAGES], (uint32_t)((j / GSTAGES) & 1), abort_flag);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == G_WARP_MMA) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
    if (tid == 0 && *abort_flag) greport(p.status, 9, 0);
}

}  // namespace
}  // namespace kad

using namespace kad;
using namespace kad::sm100;

extern "C" int kad_gemm1x1_tc_supported(int K, int N, int dtype) {
    return (dtype == KAD_F16 || dtype == KAD_BF16) && K >= 8 && K % 8 == 0 && N >= 8 && N % 8 == 0;
}

extern "C" int kad_gemm1x1_bias_act(const void* x, const void* w, const float* bias, void* y,
                                    long long M, int K, int N, int ldx, int ldy, int act, int dtype,
                                    int* status, void* stream) {
    KAD_CHECK_ARG(x && w && y && status, "kad_gemm1x1_bias_act: null pointer");
    KAD_CHECK_ARG(M > 0 && M < (1ll << 31), "kad_gemm1x1_bias_act: bad M");
    if (!kad_gemm1x1_tc_supported(K, N, dtype))
        return fail(KAD_ERR_UNSUPPORTED, "kad_gemm1x1_bias_act: needs f16/bf16, K %% 8 == 0, N %% 8 == 0 (K=%d N=%d dtype=%d)", K, N, dtype);
    KAD_CHECK_ARG(ldx >= K && ldx % 8 == 0 && ldy >= N && ldy % 8 == 0, "kad_gemm1x1_bias_act: ldx/ldy must be >= K/N and multiples of 8");
    KAD_CHECK_ARG(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)y % 16 == 0), "kad_gemm1x1_bias_act: pointers must be 16-byte aligned");
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(KAD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");

    GemmParams p{};
    p.bias = bias; p.y = y; p.status = status; p.M = M; p.K = K; p.N = N; p.ldy = ldy; p.act = act;
    p.fmt = dtype == KAD_BF16 ? 1 : 0;
    int n_tiles = (N + 255) / 256;
    int nt = ((N + n_tiles - 1) / n_tiles + 15) & ~15;
    p.nt = nt; p.n_tiles = n_tiles; p.m_tiles = (int)((M + GBM - 1) / GBM); p.ksteps = (K + 63) / 64;
    p.b_stage_bytes = nt * 128;   // multiple of 2048
    int Kp = (K + 7) & ~7;

    CUtensorMap map_a, map_b;
    CUtensorMapDataType dt = dtype == KAD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
        cuuint32_t box[2] = {64, GBM};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&map_a, dt, 2, const_cast<void*>(x), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for x failed (CUresult %d)", (int)r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        cuuint64_t strides[1] = {(cuuint64_t)Kp * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)nt};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&map_b, dt, 2, const_cast<void*>(w), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for w failed (CUresult %d)", (int)r);
    }
    // as many stages as fit in ~200 KB (4 for 256 output channels, 10 for 32): HBM-bound shapes need the bytes in flight
    const size_t fixed = sizeof(GemmBars) + (size_t)n_tiles * nt * 4 + 1024 + 128;
    // Every M tile needs the same weights: when all K slices of the (single) output-channel tile fit beside a ring of at least
    // four x stages they are loaded once per CTA and stay resident, which halves the L2 -> SM traffic of the typical layer
    // (the ring then carries x only, and gets deeper); otherwise weights stream through the ring with x.
    const size_t w_all = (size_t)p.ksteps * p.b_stage_bytes;
    const size_t budget = 224 * 1024;      // of the 227 KB a block may have
    p.resident = (n_tiles == 1 && w_all + 4 * (size_t)G_A_BYTES + fixed <= budget) ? 1 : 0;
    int stages = p.resident ? (int)((budget - fixed - w_all) / (size_t)G_A_BYTES)
                            : (int)((200 * 1024 - fixed) / (size_t)(G_A_BYTES + p.b_stage_bytes));
    stages = stages < 2 ? 2 : (stages > GMAX_STAGES ? GMAX_STAGES : stages);
    p.stages = stages;
    size_t smem = p.resident ? (size_t)stages * G_A_BYTES + w_all + fixed : (size_t)stages * (G_A_BYTES + p.b_stage_bytes) + fixed;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long ntiles = (long long)p.m_tiles * p.n_tiles;
    int grid = (int)(ntiles < sms ? ntiles : sms);
    cudaError_t e;
    if (dtype == KAD_F16) {
        auto kern = gemm1x1_tc_kernel<__half>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "gemm1x1 smem attribute: %s", cudaGetErrorString(e));
        launch_pdl(kern, grid, G_THREADS, smem, (cudaStream_t)stream, map_a, map_b, p);
    } else {
        auto kern = gemm1x1_tc_kernel<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "gemm1x1 smem attribute: %s", cudaGetErrorString(e));
        launch_pdl(kern, grid, G_THREADS, smem, (cudaStream_t)stream, map_a, map_b, p);
    }
    KAD_CHECK_LAUNCH("gemm1x1_tc_kernel");
    return KAD_OK;
}
