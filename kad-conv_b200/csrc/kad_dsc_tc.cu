// Deformable 3x3 convolution as a tcgen05 / TMEM implicit GEMM for sm_100a.
//
//   M = pixels (tiles of up to 128 pixels = th x tw image rectangle), N = Cout (<= 256), K = 9 * Cin.
//   K order: unit u = (ci / 32) * 9 + tap covers 32 input channels of one tap; a pipeline stage is
//   two units (K = 64 = one 128-byte swizzled row).
//
// One persistent CTA per SM, warp-specialised:
//   warps 0-3   epilogue: TMEM -> registers -> scale/shift/activation/post -> NHWC store (+ SE partial sums)
//   warp  4     MMA issuer (one lane): tcgen05.mma, 128 x N x 16 per instruction, fp32 accumulators in TMEM,
//               two accumulator buffers so the epilogue of tile t overlaps the MMAs of tile t+1
//   warp  5     TMA of the packed weights (B operand, 128-byte swizzle), ring of NB stages
//   warp  6     TMA of the input window: for every 32-channel chunk the tile's footprint plus a halo is
//               copied to shared memory ([wh][ww][32 ch], zero fill outside the image = zero padding),
//               double buffered
//   warps 7-22  producers: the data-dependent A operand. Per tile they first build a table of the
//               128 x 9 samples (four corner weights x mask, window address; the offsets and masks were
//               prefetched one tile ahead); then, in two groups that alternate stages, they gather the four
//               corners of every sample from the window (plain global loads for the rare sample that falls
//               outside it), interpolate, and store the 16-byte results in the swizzled K-major layout
//               the tensor core reads.
//
// All waits are time-bounded (see kad_sm100.cuh): on a timeout the CTA raises an abort flag, every
// role leaves its loop, outstanding TMA copies are waited for (bounded), TMEM is freed and the
// kernel returns with a code in the caller's status word.
#include <mutex>

#include "kad_common.cuh"
#include "kad_sm100.cuh"

namespace kad {

namespace sm100 {
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}
}  // namespace sm100

namespace {
using namespace sm100;

constexpr int BM = 128;                 // rows (pixels) per tile
constexpr int UNIT = 32;                // channels per K unit
constexpr int NA_MAX = 5;               // A stages: 3 for one CTA per tile pair, 4 for the CTA-pair kernel
constexpr int A_STAGE_BYTES = BM * 128;
constexpr int WIN_PX_MAX = 704;         // pixels per window buffer
constexpr int WIN_BYTES = WIN_PX_MAX * 64;
constexpr int NWIN = 2;
constexpr int TABLE_BYTES = BM * 9 * 16;
constexpr int EPI_WARPS = 4, PROD_WARPS = 16, PROD_GROUPS = 2, GROUP_WARPS = PROD_WARPS / PROD_GROUPS;
constexpr int WARP_MMA = 4, WARP_TMA_B = 5, WARP_TMA_WIN = 6, WARP_PROD0 = 7;
constexpr int NTHREADS_TC = (WARP_PROD0 + PROD_WARPS) * 32;   // 736
constexpr int ACC_COLS = 256;           // TMEM columns per accumulator buffer
constexpr int SMEM_LIMIT = 227 * 1024;

struct TcParams {
    const void* x; const void* offset; const void* mask;
    const float* scale; const float* shift; const float* post;
    void* y; float* gap_partial; int* status;
    int B, H, W, Cin, N;
    int th, tw, tiles_x, tiles_y, ntiles;       // tile rectangle and tile counts (per image: tiles_x*tiles_y)
    int halo, wh, ww;                           // window geometry
    int units, stages, nchunks;                 // K structure
    int na, nb, b_stage_bytes;                  // A and B rings
    int npairs;                                 // CTA-pair kernel: number of tile pairs
    int offset_f32, mask_f32, y_f32, act, fmt;
};

struct SmemLayout {
    uint32_t a, b, win, table, epi, bars;
};

// Barrier indices inside the barrier block.
struct Bars {
    uint64_t a_full[NA_MAX], a_empty[NA_MAX];
    uint64_t peer_full[NA_MAX], peer_acc[2];   // CTA-pair kernel: the peer's stage / accumulator hand-offs to the leader
    uint64_t b_full[4], b_empty[4];
    uint64_t win_full[NWIN], win_empty[NWIN];
    uint64_t acc_full[2], acc_empty[2];
    uint64_t tab_free, tab_ready;      // producer-group rendezvous around the sample table
    uint64_t gap_ready, gap_free;      // epilogue-group rendezvous around the column sums
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// r = wa*a + wb*b + wc*c + wd*d on 8 packed 16-bit channels; the weights are fp16 scalars.
template <typename T>
__device__ __forceinline__ uint4 interp8(uint4 a, uint4 b, uint4 c, uint4 d, __half wa, __half wb, __half wc, __half wd);

template <>
__device__ __forceinline__ uint4 interp8<__half>(uint4 a, uint4 b, uint4 c, uint4 d, __half wa, __half wb, __half wc, __half wd) {
    __half2 A = __half2half2(wa), Bw = __half2half2(wb), C = __half2half2(wc), D = __half2half2(wd);
    uint4 r;
    const __half2* pa = reinterpret_cast<const __half2*>(&a);
    const __half2* pb = reinterpret_cast<const __half2*>(&b);
    const __half2* pc = reinterpret_cast<const __half2*>(&c);
    const __half2* pd = reinterpret_cast<const __half2*>(&d);
    __half2* pr = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = __hfma2(D, pd[i], __hfma2(C, pc[i], __hfma2(Bw, pb[i], __hmul2(A, pa[i]))));
    return r;
}
template <>
__device__ __forceinline__ uint4 interp8<__nv_bfloat16>(uint4 a, uint4 b, uint4 c, uint4 d, __half wa, __half wb, __half wc, __half wd) {
    float fa = __half2float(wa), fb = __half2float(wb), fc = __half2float(wc), fd = __half2float(wd);
    uint4 r;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&c);
    const __nv_bfloat162* pd = reinterpret_cast<const __nv_bfloat162*>(&d);
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 va = __bfloat1622float2(pa[i]), vb = __bfloat1622float2(pb[i]);
        float2 vc = __bfloat1622float2(pc[i]), vd = __bfloat1622float2(pd[i]);
        float lo = fmaf(fd, vd.x, fmaf(fc, vc.x, fmaf(fb, vb.x, fa * va.x)));
        float hi = fmaf(fd, vd.y, fmaf(fc, vc.y, fmaf(fb, vb.y, fa * va.y)));
        pr[i] = __floats2bfloat162_rn(lo, hi);
    }
    return r;
}

__device__ __forceinline__ void report(int* status, int code, int detail) {
    if (atomicCAS(status, 0, code) == 0) { status[1] = detail; status[2] = blockIdx.x; }
}

// Rendezvous of a warp group on an mbarrier whose count is the number of warps: bounded like every wait.
__device__ __forceinline__ bool group_sync(uint64_t* bar, uint32_t parity, int lane, volatile int* abort_flag) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    return mbar_wait(bar, parity, abort_flag);
}

// AFFINE: the epilogue applies scale/shift/activation/post; otherwise it only converts and stores.
template <typename T, bool AFFINE, bool PAIR>
__global__ void __launch_bounds__(NTHREADS_TC, 1)
dsc_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
              const TcParams p, const SmemLayout L) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);   // swizzled tiles need 1024-byte alignment
    Bars* bars = reinterpret_cast<Bars*>(smem + L.bars);
    volatile int* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_per_img = p.tiles_x * p.tiles_y;
    const uint32_t NA = (uint32_t)p.na;
    // Tile schedule. One CTA per SM: CTA c takes tiles c, c + grid, ... In the CTA-pair kernel the two CTAs of cluster q
    // take tiles 2k and 2k+1 of pair k = q, q + clusters, ...; the last pair may hold one tile past the end, which is
    // produced as zeros and not stored.
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int sched0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, sched_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int sched_n = PAIR ? p.npairs : p.ntiles;
    const int niter = sched0 < sched_n ? (sched_n - sched0 + sched_step - 1) / sched_step : 0;
    auto tile_at = [&](int it_) { const int k = sched0 + it_ * sched_step; return PAIR ? 2 * k + (int)rank : k; };

    if (tid == 0) {
        // CTA pair: the peer's producers arrive directly on the leader's a_full (8 local + 8 remote warps per stage)
        for (int i = 0; i < NA_MAX; ++i) { mbar_init(&bars->a_full[i], PAIR ? 2 * GROUP_WARPS : GROUP_WARPS); mbar_init(&bars->a_empty[i], 1); mbar_init(&bars->peer_full[i], 1); }
        for (int i = 0; i < 2; ++i) mbar_init(&bars->peer_acc[i], 1);
        for (int i = 0; i < 4; ++i) { mbar_init(&bars->b_full[i], 1); mbar_init(&bars->b_empty[i], 1); }
        for (int i = 0; i < NWIN; ++i) { mbar_init(&bars->win_full[i], 1); mbar_init(&bars->win_empty[i], PROD_WARPS); }
        for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 1); mbar_init(&bars->acc_empty[i], EPI_WARPS * 32); }
        mbar_init(&bars->tab_free, PROD_WARPS); mbar_init(&bars->tab_ready, PROD_WARPS);
        mbar_init(&bars->gap_ready, EPI_WARPS); mbar_init(&bars->gap_free, EPI_WARPS);
        bars->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == WARP_MMA) {
        if (PAIR) { tmem_alloc_pair(&bars->tmem_base, 512); tmem_relinquish_pair(); }
        else { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
    }
    // epilogue parameters: scale | shift | post, float[256] each
    float* epi = reinterpret_cast<float*>(smem + L.epi);
    for (int i = tid; i < 256; i += NTHREADS_TC) {
        bool live = i < p.N;
        epi[i] = (live && p.scale) ? p.scale[i] : 1.f;
        epi[256 + i] = (live && p.shift) ? p.shift[i] : 0.f;
        epi[512 + i] = (live && p.post) ? p.post[i] : 1.f;
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();     // the peer's barriers exist before anything arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp < EPI_WARPS) {
        // =========================================================================== epilogue
        float* gsum = epi + 768;   // [4 warps][256] column sums for the SE squeeze
        int it = 0;
        for (; it < niter; ++it) {
            const int tile_raw = tile_at(it);
            const bool tile_ok = tile_raw < p.ntiles;
            const int tile = tile_ok ? tile_raw : p.ntiles - 1;
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_full[buf], (it >> 1) & 1, abort_flag)) { report(p.status, 1, it); break; }
            tc_fence_after();
            const int b = tile / tiles_per_img, tr = tile - b * tiles_per_img;
            const int ty0 = (tr / p.tiles_x) * p.th, tx0 = (tr % p.tiles_x) * p.tw;
            const int r = warp * 32 + lane;
            const int ry = r / p.tw, rx = r - ry * p.tw;
            const int py = ty0 + ry, px = tx0 + rx;
            const bool live = tile_ok && (r < p.th * p.tw) && py < p.H && px < p.W;
            const size_t obase = (((size_t)b * p.H + py) * p.W + px) * p.N;
            for (int c0 = 0; c0 < p.N; c0 += 32) {
                const int nc = min(32, p.N - c0);   // 32 or 16
                uint32_t v[32];
                const uint32_t taddr = tmem_base + (uint32_t)(buf * ACC_COLS + c0) + ((uint32_t)(warp * 32) << 16);
                if (nc == 32) tmem_ld_32x32(taddr, v); else tmem_ld_32x16(taddr, v);
                tmem_ld_wait();
                float o[32];
                if (AFFINE) {
                    const float4* sc4 = reinterpret_cast<const float4*>(epi + c0);
                    const float4* sh4 = reinterpret_cast<const float4*>(epi + 256 + c0);
                    const float4* po4 = reinterpret_cast<const float4*>(epi + 512 + c0);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4) {
                        const float4 sc = sc4[q4], sh = sh4[q4], po = po4[q4];
                        o[4 * q4 + 0] = apply_act(fmaf(__uint_as_float(v[4 * q4 + 0]), sc.x, sh.x), p.act) * po.x;
                        o[4 * q4 + 1] = apply_act(fmaf(__uint_as_float(v[4 * q4 + 1]), sc.y, sh.y), p.act) * po.y;
                        o[4 * q4 + 2] = apply_act(fmaf(__uint_as_float(v[4 * q4 + 2]), sc.z, sh.z), p.act) * po.z;
                        o[4 * q4 + 3] = apply_act(fmaf(__uint_as_float(v[4 * q4 + 3]), sc.w, sh.w), p.act) * po.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(v[j]);
                }
                if (live) {
                    if (p.y_f32) {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + obase + c0);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (j * 4 < nc) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.y) + obase + c0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (j * 8 < nc) {
                                uint4 w;
                                T* h = reinterpret_cast<T*>(&w);
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = from_f<T>(o[8 * j + e]);
                                dst[j] = w;
                            }
                        }
                    }
                }
                if (p.gap_partial) {
                    // column sums over the warp's 32 rows: butterfly that halves the columns per lane each step
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = (live && j < nc) ? (p.y_f32 ? o[j] : to_f<T>(from_f<T>(o[j]))) : 0.f;
#pragma unroll
                    for (int step = 16; step >= 1; step >>= 1) {
                        const bool upper = (lane & step) != 0;
#pragma unroll
                        for (int j = 0; j < step; ++j) {
                            float send = upper ? o[j] : o[j + step];
                            float keep = upper ? o[j + step] : o[j];
                            o[j] = keep + __shfl_xor_sync(0xffffffffu, send, step);
                        }
                    }
                    if (lane < nc) gsum[warp * 256 + c0 + lane] = o[0];   // lane l ends up with column l
                }
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[buf]);
            if (p.gap_partial && tile_ok) {
                if (!group_sync(&bars->gap_ready, it & 1, lane, abort_flag)) { report(p.status, 10, it); break; }
                for (int c = tid; c < p.N; c += EPI_WARPS * 32)
                    p.gap_partial[((size_t)b * tiles_per_img + tr) * p.N + c] =
                        gsum[c] + gsum[256 + c] + gsum[512 + c] + gsum[768 + c];
                if (!group_sync(&bars->gap_free, it & 1, lane, abort_flag)) { report(p.status, 11, it); break; }
            }
        }
    } else if (warp == WARP_MMA) {
        // =========================================================================== MMA issuer
        // This warp's instruction stream is one dependent chain per stage (nothing else hides its latency), so the loop
        // keeps ring slots and phases in wrapping counters (no divisions) and the operand descriptors precomputed.
        const uint32_t idesc = PAIR ? instr_desc_f16_pair(p.fmt, p.N) : instr_desc_f16(p.fmt, p.N);
        const uint64_t adesc0 = smem_desc_sw128(smem_u32(smem + L.a)), bdesc0 = smem_desc_sw128(smem_u32(smem + L.b));
        const uint32_t a_step = A_STAGE_BYTES >> 4, b_step = (uint32_t)p.b_stage_bytes >> 4;   // descriptor address units of 16 bytes
        const uint32_t nbr = (uint32_t)p.nb;
        uint32_t sa = 0, pa = 0, sb = 0, pb = 0;     // slot and phase parity of the A and B rings
        bool ok = true;
        for (int it = 0; it < niter && ok; ++it) {
            const int buf = it & 1;
            if (!mbar_wait(&bars->acc_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag)) { report(p.status, 2, it); break; }
            if (PAIR) {
                // the leader also needs the peer's accumulator buffer drained; the peer's MMA warp passes that on
                if (rank == 1) { __syncwarp(); if (lane == 0) mbar_arrive_remote(&bars->peer_acc[buf], 0); }
                else if (!mbar_wait_cluster(&bars->peer_acc[buf], (it >> 1) & 1, abort_flag)) { report(p.status, 14, it); break; }
            }
            tc_fence_after();
            const uint32_t tacc = tmem_base + (uint32_t)(buf * ACC_COLS);
            const int last = p.stages - 1;
            const int nk_last = (p.units & 1) ? 2 : 4;   // a trailing single unit fills half a stage
            for (int s = 0; s <= last; ++s) {
                // lane 0 waits for the A stage, lane 1 for the B stage (lane 2: the peer's stage): the waits overlap
                bool okw = true;
                if (lane == 0 && !(PAIR && rank == 1)) {      // A stage (both CTAs' halves in pair mode)
                    okw = PAIR ? mbar_wait_cluster(&bars->a_full[sa], pa, abort_flag) : mbar_wait(&bars->a_full[sa], pa, abort_flag);
                } else if (lane == 1) { okw = mbar_wait(&bars->b_full[sb], pb, abort_flag); }
                else if (PAIR && lane == 2 && rank == 0) { okw = mbar_wait_cluster(&bars->peer_full[sa], pa, abort_flag); }
                if (!__all_sync(0xffffffffu, okw)) { report(p.status, 3, s); ok = false; break; }
                // no tcgen05 fence here: the operands come through shared memory (mbarrier + proxy fence order them);
                // only the accumulator hand-off above involves TMEM
                if (PAIR && rank == 1) {
                    // peer CTA: its half of the weights for this stage has landed; tell the leader, which issues for both
                    if (lane == 0) mbar_arrive_remote(&bars->peer_full[sa], 0);
                } else if (lane == 0) {
                    const uint64_t ad = adesc0 + (uint64_t)(sa * a_step), bd = bdesc0 + (uint64_t)(sb * b_step);
                    const int nk = (s == last) ? nk_last : 4;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (k < nk) {
                            if (PAIR) umma_f16_pair(tacc, ad + 2u * k, bd + 2u * k, idesc, (s | k) ? 1u : 0u);
                            else umma_f16(tacc, ad + 2u * k, bd + 2u * k, idesc, (s | k) ? 1u : 0u);
                        }
                    }
                    if (PAIR) {
                        umma_commit_pair(&bars->a_empty[sa]);
                        if (s == last) umma_commit_pair(&bars->acc_full[buf]);
                    } else {
                        umma_commit(&bars->a_empty[sa]);
                        if (s == last) umma_commit(&bars->acc_full[buf]);
                    }
                }
                if (++sa == NA) { sa = 0; pa ^= 1; }
                if (++sb == nbr) { sb = 0; pb ^= 1; }
                __syncwarp();
            }
        }
    } else if (warp == WARP_TMA_B) {
        // =========================================================================== weights
        if (lane == 0) {
            tma_prefetch_desc(&map_w);
            uint32_t ib = 0, sb = 0;
            uint32_t ja = 0, jp = 0;                  // ring slot / phase parity of the stage whose completion frees the slot
            const uint32_t nbr = (uint32_t)p.nb;
            bool ok = true;
            for (int it = 0; it < niter && ok; ++it) {
                for (int s = 0; s < p.stages; ++s, ++ib) {
                    if (ib >= nbr) {
                        // The slot is free once the MMAs of stage j = ib - nb are done. That is the event the A ring's
                        // a_empty[j % NA] barrier already records (one tcgen05.commit per stage serves both rings); with
                        // nb <= NA that barrier cannot run a further phase ahead before this load is issued.
                        if (!mbar_wait(&bars->a_empty[ja], jp, abort_flag)) { report(p.status, 5, s); ok = false; break; }
                        if (++ja == NA) { ja = 0; jp ^= 1u; }
                    }
                    mbar_arrive_expect_tx(&bars->b_full[sb], (uint32_t)p.b_stage_bytes);
                    tma_load_2d(smem + L.b + sb * p.b_stage_bytes, &map_w, 0, s * p.N + (PAIR ? (int)rank * (p.N >> 1) : 0), &bars->b_full[sb]);
                    if (++sb == nbr) sb = 0;
                }
            }
            if (!ok || *abort_flag) {   // let copies in flight land before the CTA goes away
                for (uint32_t i = 0; i < (uint32_t)p.nb && i < ib; ++i) {
                    uint32_t j = ib - 1 - i;
                    mbar_wait(&bars->b_full[j % (uint32_t)p.nb], (j / (uint32_t)p.nb) & 1, abort_flag);
                }
            }
        }
    } else if (warp == WARP_TMA_WIN) {
        // =========================================================================== input windows
        if (lane == 0) {
            tma_prefetch_desc(&map_x);
            uint32_t iw = 0;
            bool ok = true;
            const uint32_t win_bytes = (uint32_t)(p.wh * p.ww * 64);
            for (int it = 0; it < niter && ok; ++it) {
                const int tile = min(tile_at(it), p.ntiles - 1);
                const int b = tile / tiles_per_img, tr = tile - b * tiles_per_img;
                const int wy0 = (tr / p.tiles_x) * p.th - 1 - p.halo, wx0 = (tr % p.tiles_x) * p.tw - 1 - p.halo;
                for (int cc = 0; cc < p.nchunks; ++cc, ++iw) {
                    const uint32_t sw = iw % NWIN;
                    if (!mbar_wait(&bars->win_empty[sw], ((iw / NWIN) & 1) ^ 1, abort_flag)) { report(p.status, 6, cc); ok = false; break; }
                    mbar_arrive_expect_tx(&bars->win_full[sw], win_bytes);
                    tma_load_4d(smem + L.win + sw * WIN_BYTES, &map_x, cc * UNIT, wx0, wy0, b, &bars->win_full[sw]);
                }
            }
            if (!ok || *abort_flag) {
                for (uint32_t i = 0; i < NWIN && i < iw; ++i) {
                    uint32_t j = iw - 1 - i;
                    mbar_wait(&bars->win_full[j % NWIN], (j / NWIN) & 1, abort_flag);
                }
            }
        }
    } else {
        // =========================================================================== producers
        // 16 warps in two groups of 8; group g fills the stages s = g, g+2, ... so that the per-stage latency
        // (barrier wait, gather, proxy fence) of one group overlaps the other group's stage.
        const int pw = warp - WARP_PROD0;            // 0..15
        const int grp = pw / GROUP_WARPS, pwg = pw % GROUP_WARPS;
        const int ptid = tid - WARP_PROD0 * 32;      // 0..511
        const int sub = lane & 3, g = (lane >> 2) & 1, q = lane >> 3;
        const int rloc = pwg * 8 + g * 4 + q;        // row within a 64-row pass; (row >> 2) & 1 == g
        const uint32_t a_base = smem_u32(smem + L.a), win_base = smem_u32(smem + L.win), tab_base = smem_u32(smem + L.table);
        uint4* table = reinterpret_cast<uint4*>(smem + L.table);
        const uint32_t rowpitch = (uint32_t)p.ww * 64;
        // per-thread constants of its two rows (pass 0 / 1): table row base and swizzled store offsets per unit slot
        uint32_t tab_row[2], st_off[2][2];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
            const int row = pass * 64 + rloc;
            tab_row[pass] = tab_base + (uint32_t)(row * 9) * 16;
#pragma unroll
            for (int j = 0; j < 2; ++j) st_off[pass][j] = (uint32_t)row * 128 + (uint32_t)(((j * 4 + sub) ^ (row & 7)) << 4);
        }
        constexpr int TAB_ITERS = (BM * 9 + PROD_WARPS * 32 - 1) / (PROD_WARPS * 32);   // 3
        float pf[TAB_ITERS][3];                      // offsets (dy, dx) and mask of this thread's table entries

        // loads the raw sample parameters of a tile into registers (issued one tile ahead)
        auto prefetch = [&](int tile_) {
            const int b_ = tile_ / tiles_per_img, tr_ = tile_ - b_ * tiles_per_img;
            const int ty0_ = (tr_ / p.tiles_x) * p.th, tx0_ = (tr_ % p.tiles_x) * p.tw;
#pragma unroll
            for (int i = 0; i < TAB_ITERS; ++i) {
                const int e = ptid + i * PROD_WARPS * 32;
                pf[i][0] = 0.f; pf[i][1] = 0.f; pf[i][2] = 1.f;
                if (e < BM * 9 && tile_ < p.ntiles && tile_ >= 0) {
                    const int r = e / 9, k = e - r * 9;
                    const int ry = r / p.tw, rx = r - ry * p.tw;
                    const int py = ty0_ + ry, px = tx0_ + rx;
                    if (r < p.th * p.tw && py < p.H && px < p.W) {
                        const size_t pix = ((size_t)b_ * p.H + py) * p.W + px;
                        if (p.offset) { pf[i][0] = load_mixed<T>(p.offset, pix * 18 + 2 * k, p.offset_f32); pf[i][1] = load_mixed<T>(p.offset, pix * 18 + 2 * k + 1, p.offset_f32); }
                        if (p.mask) pf[i][2] = load_mixed<T>(p.mask, pix * 9 + k, p.mask_f32);
                    }
                }
            }
        };

        bool ok = true;
        int it = 0;
        uint32_t cur_ia = 0, sa = 0, pa = 0;          // stage counter of this group and its ring slot / phase parity
        prefetch(niter > 0 ? tile_at(0) : -1);
        for (; it < niter && ok; ++it) {
            const int tile_raw = tile_at(it);
            const bool tile_ok = tile_raw < p.ntiles;
            const int tile = tile_ok ? tile_raw : p.ntiles - 1;
            const int b = tile / tiles_per_img, tr = tile - b * tiles_per_img;
            const int ty0 = (tr / p.tiles_x) * p.th, tx0 = (tr % p.tiles_x) * p.tw;
            const int wy0 = ty0 - 1 - p.halo, wx0 = tx0 - 1 - p.halo;
            // everybody is done reading the previous table
            if (!group_sync(&bars->tab_free, it & 1, lane, abort_flag)) { report(p.status, 12, it); break; }
            // ---- sample table [row][tap] -> {w_first|w_second, w_first_below|w_second_below, window offset|flags, y0<<16|x0}
            // The 'first' corner is the one whose window pixel parity equals the row's group bit, so that the two rows
            // a quarter-warp reads together touch different halves of the shared-memory banks (ww is even).
            // flags: bit 0 = second corner lies 64 bytes before the first; bit 1 = sample outside the window (global path).
#pragma unroll
            for (int i = 0; i < TAB_ITERS; ++i) {
                const int e = ptid + i * PROD_WARPS * 32;
                if (e < BM * 9) {
                    const int r = e / 9, k = e - r * 9;
                    const int ry = r / p.tw, rx = r - ry * p.tw;
                    const int py = ty0 + ry, px = tx0 + rx;
                    float w00 = 0.f, w01 = 0.f, w10 = 0.f, w11 = 0.f;
                    uint32_t word = 0, pos = 0;
                    if (tile_ok && r < p.th * p.tw && py < p.H && px < p.W) {
                        const float sy = (float)(py + k / 3 - 1) + pf[i][0], sx = (float)(px + k % 3 - 1) + pf[i][1];
                        if (sy > -1.f && sy < (float)p.H && sx > -1.f && sx < (float)p.W) {
                            const float m = pf[i][2];
                            const float fy = floorf(sy), fx = floorf(sx);
                            const int y0 = (int)fy, x0 = (int)fx;
                            const float ly = sy - fy, lx = sx - fx, hy = 1.f - ly, hx = 1.f - lx;
                            w00 = hy * hx * m; w01 = hy * lx * m; w10 = ly * hx * m; w11 = ly * lx * m;
                            const int wy = y0 - wy0, wx = x0 - wx0;
                            if (wy >= 0 && wy + 1 < p.wh && wx >= 0 && wx + 1 < p.ww) {
                                const uint32_t addr = (uint32_t)(wy * p.ww + wx) * 64;
                                if ((int)((addr >> 6) & 1) != ((r >> 2) & 1)) {      // start with the right-hand corner
                                    word = (addr + 64) | 1u;
                                    float t = w00; w00 = w01; w01 = t; t = w10; w10 = w11; w11 = t;
                                } else {
                                    word = addr;
                                }
                            } else {
                                word = 2u; pos = ((uint32_t)y0 << 16) | ((uint32_t)x0 & 0xffffu);
                            }
                        }
                    }
                    __half2 wa = __floats2half2_rn(w00, w01), wb = __floats2half2_rn(w10, w11);
                    uint4 ent;
                    ent.x = *reinterpret_cast<uint32_t*>(&wa); ent.y = *reinterpret_cast<uint32_t*>(&wb);
                    ent.z = word; ent.w = pos;
                    table[e] = ent;
                }
            }
            if (!group_sync(&bars->tab_ready, it & 1, lane, abort_flag)) { report(p.status, 13, it); break; }
            prefetch(it + 1 < niter ? tile_at(it + 1) : -1);   // next tile's offsets and mask arrive while this tile is gathered

            int have_cc = -1;                        // chunks whose window this thread has already waited for
            const uint32_t ia0 = (uint32_t)it * (uint32_t)p.stages, iw0 = (uint32_t)it * (uint32_t)p.nchunks;
            for (int s = grp; s < p.stages && ok; s += PROD_GROUPS) {
                {   // move the ring position (slot sa, phase parity pa) forward to this stage without dividing
                    const uint32_t target = ia0 + (uint32_t)s;
                    sa += target - cur_ia; cur_ia = target;
                    while (sa >= NA) { sa -= NA; pa ^= 1u; }
                }
                if (!mbar_wait(&bars->a_empty[sa], pa ^ 1u, abort_flag)) { report(p.status, 7, s); ok = false; break; }
                const uint32_t a_stage = a_base + sa * A_STAGE_BYTES;
                const int nu = (2 * s + 1 < p.units) ? 2 : 1;     // a trailing single unit is produced twice (harmless)
                int tapj[2], ccj[2];
                uint32_t winj[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int u = 2 * s + (j < nu ? j : 0);
                    ccj[j] = u / 9; tapj[j] = u - ccj[j] * 9;
                    const uint32_t iwc = iw0 + (uint32_t)ccj[j];     // window counter of this chunk
                    const uint32_t sw = iwc % NWIN;
                    if (ccj[j] > have_cc) {          // first use of this chunk: its window must have landed
                        if (!mbar_wait(&bars->win_full[sw], (iwc / NWIN) & 1, abort_flag)) { report(p.status, 8, u); ok = false; }
                        have_cc = ccj[j];
                    }
                    winj[j] = win_base + sw * WIN_BYTES + sub * 16;
                }
                if (!ok) break;
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
                    // two independent tasks (the stage's two units of one row): table reads, then eight corner
                    // loads, then the arithmetic
                    uint4 ent[2], v[2][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j) ent[j] = lds128(tab_row[pass] + (uint32_t)tapj[j] * 16);
                    const bool slow = ((ent[0].z | ent[1].z) & 2u) != 0;
                    if (!__any_sync(0xffffffffu, slow)) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t first = winj[j] + (ent[j].z & ~63u);
                            const uint32_t second = first + 64u - ((ent[j].z & 1u) << 7);
                            v[j][0] = lds128(first); v[j][1] = lds128(second);
                            v[j][2] = lds128(first + rowpitch); v[j][3] = lds128(second + rowpitch);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (!(ent[j].z & 2u)) {
                                const uint32_t first = winj[j] + (ent[j].z & ~63u);
                                const uint32_t second = first + 64u - ((ent[j].z & 1u) << 7);
                                v[j][0] = lds128(first); v[j][1] = lds128(second);
                                v[j][2] = lds128(first + rowpitch); v[j][3] = lds128(second + rowpitch);
                            } else {
                                const uint32_t pos = ent[j].w;
                                const int y0 = (int)pos >> 16, x0 = (int)(short)(pos & 0xffff);
                                const T* xb = reinterpret_cast<const T*>(p.x) + (size_t)b * p.H * p.W * p.Cin + ccj[j] * UNIT + sub * 8;
                                const uint4 z = make_uint4(0, 0, 0, 0);
                                const bool y0ok = y0 >= 0, y1ok = y0 + 1 < p.H, x0ok = x0 >= 0, x1ok = x0 + 1 < p.W;
                                v[j][0] = (y0ok && x0ok) ? ldg128(xb + ((ptrdiff_t)y0 * p.W + x0) * p.Cin) : z;
                                v[j][1] = (y0ok && x1ok) ? ldg128(xb + ((ptrdiff_t)y0 * p.W + x0 + 1) * p.Cin) : z;
                                v[j][2] = (y1ok && x0ok) ? ldg128(xb + ((ptrdiff_t)(y0 + 1) * p.W + x0) * p.Cin) : z;
                                v[j][3] = (y1ok && x1ok) ? ldg128(xb + ((ptrdiff_t)(y0 + 1) * p.W + x0 + 1) * p.Cin) : z;
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const __half2 wa = *reinterpret_cast<const __half2*>(&ent[j].x), wb = *reinterpret_cast<const __half2*>(&ent[j].y);
                        const uint4 res = interp8<T>(v[j][0], v[j][1], v[j][2], v[j][3], __low2half(wa), __high2half(wa),
                                                     __low2half(wb), __high2half(wb));
                        sts128(a_stage + st_off[pass][j], res);
                    }
                }
                // release a chunk's window after this group's last stage that reads it
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (j < nu && (j == nu - 1 || ccj[j + 1 < 2 ? j + 1 : j] != ccj[j])) {
                        const int Lc = (9 * ccj[j] + 8) >> 1;                 // last stage holding a unit of the chunk
                        const int Lg = Lc - ((Lc - grp) & 1);                 // ... that belongs to this group
                        if (s == Lg) {
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&bars->win_empty[(iw0 + (uint32_t)ccj[j]) % NWIN]);
                        }
                    }
                }
                fence_proxy_async();                             // generic-proxy stores -> visible to the tensor core
                __syncwarp();
                if (lane == 0) { if (PAIR && rank == 1) mbar_arrive_remote(&bars->a_full[sa], 0); else mbar_arrive(&bars->a_full[sa]); }
            }
        }
    }

    // ------------------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();     // the leader's MMAs read the peer's shared memory: leave together
    if (warp == WARP_MMA) { tc_fence_after(); if (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512); }
    if (tid == 0 && *abort_flag) report(p.status, 9, 0);
}

template <typename T>
__global__ void pack_weight_tc_kernel(const float* __restrict__ w, T* __restrict__ dst, int Cin, int Cout, int stages) {
    // dst[s][n][j]: K index kk = s*64 + j -> unit u = kk/32 (cc = u/9, tap = u%9), channel ci = cc*32 + kk%32
    size_t n = (size_t)stages * Cout * 64;
    int units = 9 * (Cin / UNIT);
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        int j = (int)(e % 64);
        size_t r = e / 64;
        int o = (int)(r % Cout), s = (int)(r / Cout);
        int kk = s * 64 + j, u = kk / UNIT;
        float v = 0.f;
        if (u < units) {
            int cc = u / 9, tap = u - cc * 9, ci = cc * UNIT + kk % UNIT;
            v = w[((size_t)o * Cin + ci) * 9 + tap];
        }
        dst[e] = from_f<T>(v);
    }
}

struct TileChoice { int th, tw, halo, wh, ww; };

// Tile rectangle with th*tw <= 128 that covers the image with the fewest tiles; the window
// (tile + taps + halo + 1, width rounded to even) must fit one window buffer.
TileChoice choose_tile(int H, int W) {
    TileChoice best{0, 0, 0, 0, 0};
    long long best_cost = -1;
    for (int th = 1; th <= H && th <= BM; ++th) {
        int tw = BM / th;
        if (tw > W) tw = W;
        if (tw < 1) continue;
        int halo = -1, wh = 0, ww = 0;
        for (int h = 8; h >= 1; --h) {
            int a = th + 2 * h + 2, bb = (tw + 2 * h + 2 + 1) & ~1;
            if (a * bb <= WIN_PX_MAX && a <= 256 && bb <= 256) { halo = h; wh = a; ww = bb; break; }
        }
        if (halo < 1) continue;
        long long tiles = (long long)((H + th - 1) / th) * ((W + tw - 1) / tw);
        // fewer tiles first; a small halo sends more samples down the slow path, so penalise it
        long long cost = tiles * 16 + (halo >= 5 ? 0 : (5 - halo) * 4 * tiles / 4);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = {th, tw, halo, wh, ww}; }
    }
    return best;
}

}  // namespace

int dsc_tc_tiles(int H, int W) {
    TileChoice t = choose_tile(H, W);
    if (t.th == 0) return 0;
    return ((H + t.th - 1) / t.th) * ((W + t.tw - 1) / t.tw);
}

int launch_dsc_tc(const KadDscArgs& a, cudaStream_t st) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(KAD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    KAD_CHECK_ARG(((uintptr_t)a.x % 16 == 0) && ((uintptr_t)a.weight % 16 == 0) && ((uintptr_t)a.y % 16 == 0),
                  "kad_dsc_forward: x, weight and y must be 16-byte aligned for the tensor path");
    KAD_CHECK_ARG(a.H <= 32767 && a.W <= 32767, "kad_dsc_forward: image side above 32767");
    TileChoice t = choose_tile(a.H, a.W);
    KAD_CHECK_ARG(t.th > 0, "kad_dsc_forward: no tile shape for %dx%d", a.H, a.W);

    TcParams p{};
    p.x = a.x; p.offset = a.offset; p.mask = a.mask; p.scale = a.scale; p.shift = a.shift; p.post = a.post;
    p.y = a.y; p.gap_partial = a.gap_partial; p.status = a.status;
    p.B = a.B; p.H = a.H; p.W = a.W; p.Cin = a.Cin; p.N = a.Cout;
    p.th = t.th; p.tw = t.tw; p.halo = t.halo; p.wh = t.wh; p.ww = t.ww;
    p.tiles_x = (a.W + t.tw - 1) / t.tw; p.tiles_y = (a.H + t.th - 1) / t.th;
    long long nt = (long long)p.tiles_x * p.tiles_y * a.B;
    KAD_CHECK_ARG(nt < (1ll << 31), "kad_dsc_forward: too many tiles");
    p.ntiles = (int)nt;
    p.nchunks = a.Cin / UNIT; p.units = 9 * p.nchunks; p.stages = (p.units + 1) / 2;
    p.b_stage_bytes = a.Cout * 128;
    p.offset_f32 = a.offset_f32; p.mask_f32 = a.mask_f32; p.y_f32 = a.y_f32; p.act = a.act;
    p.fmt = a.dtype == KAD_BF16 ? 1 : 0;

    // One CTA per tile, or a CTA pair (cluster of 2, tcgen05 cta_group::2) per two tiles: the pair splits the weight
    // operand by N between the two CTAs' shared memories, which halves the weight bytes every SM has to stage.
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // path 2 selects the pair kernel. It is not what path 1 uses: on C1 it measured 370-380 us against 310-320 us for
    // one CTA per tile, because the weight ring and the hand-off between the two CTAs add latency that the four A
    // stages which fit in shared memory do not cover.
    const bool pair = a.path == 2;
    if (pair) KAD_CHECK_ARG(a.Cout % 32 == 0 && p.ntiles >= 2 && sms >= 2, "kad_dsc_forward: the CTA-pair kernel needs Cout %% 32 == 0 and at least two tiles");
    p.npairs = (p.ntiles + 1) / 2;
    p.na = pair ? 4 : 3;
    p.b_stage_bytes = (pair ? a.Cout / 2 : a.Cout) * 128;      // multiple of 2048

    // shared-memory carve-up (offsets from a 1024-byte aligned base)
    SmemLayout L{};
    uint32_t off = 0;
    L.a = off; off += p.na * A_STAGE_BYTES;
    L.b = off;
    uint32_t fixed_after = NWIN * WIN_BYTES + TABLE_BYTES + (768 + 1024) * 4 + 1024;
    int nb = (int)((SMEM_LIMIT - 1024 - (int)off - (int)fixed_after) / p.b_stage_bytes);
    if (nb > p.na) nb = p.na;   // the weight ring is released through the A ring's barriers, which needs nb <= na
    KAD_CHECK_ARG(nb >= 2, "kad_dsc_forward: no room for two weight stages");
    p.nb = nb;
    off += nb * p.b_stage_bytes;
    L.win = off; off += NWIN * WIN_BYTES;
    L.table = off; off += TABLE_BYTES;
    L.epi = off; off += (768 + 1024) * 4;
    L.bars = off; off += 1024;
    size_t smem = off + 1024;   // slack for the runtime alignment of the dynamic segment

    // tensor maps
    CUtensorMap map_x, map_w;
    CUtensorMapDataType dt = a.dtype == KAD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    {
        cuuint64_t dims[4] = {(cuuint64_t)a.Cin, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.B};
        cuuint64_t strides[3] = {(cuuint64_t)a.Cin * 2, (cuuint64_t)a.W * a.Cin * 2, (cuuint64_t)a.H * a.W * a.Cin * 2};
        cuuint32_t box[4] = {(cuuint32_t)UNIT, (cuuint32_t)t.ww, (cuuint32_t)t.wh, 1};
        cuuint32_t es[4] = {1, 1, 1, 1};
        CUresult r = enc(&map_x, dt, 4, const_cast<void*>(a.x), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for x failed (CUresult %d)", (int)r);
    }
    {
        cuuint64_t dims[2] = {64, (cuuint64_t)p.stages * a.Cout};
        cuuint64_t strides[1] = {128};
        cuuint32_t box[2] = {64, (cuuint32_t)(pair ? a.Cout / 2 : a.Cout)};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(&map_w, dt, 2, const_cast<void*>(a.weight), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(KAD_ERR_CUDA, "tensor map for the weights failed (CUresult %d)", (int)r);
    }

    const bool affine = a.scale || a.shift || a.post || a.act != KAD_ACT_NONE;
    void (*kern)(const CUtensorMap, const CUtensorMap, const TcParams, const SmemLayout);
    if (a.dtype == KAD_F16) {
        kern = pair ? (affine ? dsc_tc_kernel<__half, true, true> : dsc_tc_kernel<__half, false, true>)
                    : (affine ? dsc_tc_kernel<__half, true, false> : dsc_tc_kernel<__half, false, false>);
    } else {
        kern = pair ? (affine ? dsc_tc_kernel<__nv_bfloat16, true, true> : dsc_tc_kernel<__nv_bfloat16, false, true>)
                    : (affine ? dsc_tc_kernel<__nv_bfloat16, true, false> : dsc_tc_kernel<__nv_bfloat16, false, false>);
    }
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_tc smem attribute (%zu bytes): %s", smem, cudaGetErrorString(e));
    if (pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (sms / 2)); cfg.blockDim = dim3(NTHREADS_TC); cfg.dynamicSmemBytes = smem; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        // The schedule is static and every CTA needs a whole SM: launch only as many pairs as can be resident together
        // (an SM whose partner is unavailable cannot host a pair), otherwise the excess pairs would run as a second wave.
        static int resident_pairs[64][2] = {};
        int& cached = resident_pairs[dev < 64 ? dev : 0][affine ? 1 : 0];
        if (cached == 0) {
            int n = 0;
            cudaError_t eq = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
            cached = (eq == cudaSuccess && n > 0) ? n : sms / 2;
        }
        int clusters = p.npairs < cached ? p.npairs : cached;
        cfg.gridDim = dim3(2 * clusters);
        e = cudaLaunchKernelEx(&cfg, kern, map_x, map_w, p, L);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_tc_kernel (CTA pair) launch: %s", cudaGetErrorString(e));
    } else {
        int grid = p.ntiles < sms ? p.ntiles : sms;
        kern<<<grid, NTHREADS_TC, smem, st>>>(map_x, map_w, p, L);
    }
    KAD_CHECK_LAUNCH("dsc_tc_kernel");
    return KAD_OK;
}

}  // namespace kad

using namespace kad;

extern "C" int kad_dsc_tc_supported(int Cin, int Cout, int dtype) {
    return (dtype == KAD_F16 || dtype == KAD_BF16) && Cin > 0 && Cin % 32 == 0 && Cout >= 16 && Cout % 16 == 0 && Cout <= 256;
}

extern "C" size_t kad_dsc_packed_weight_bytes(int Cin, int Cout, int dtype) {
    if (!kad_dsc_tc_supported(Cin, Cout, dtype)) return 0;
    int units = 9 * (Cin / 32), stages = (units + 1) / 2;
    return (size_t)stages * Cout * 64 * 2;
}

extern "C" int kad_dsc_pack_weight_tc(const float* w_oihw, void* dst, int Cin, int Cout, int dtype, void* stream) {
    KAD_CHECK_ARG(w_oihw && dst, "kad_dsc_pack_weight_tc: null pointer");
    if (!kad_dsc_tc_supported(Cin, Cout, dtype)) return fail(KAD_ERR_UNSUPPORTED, "kad_dsc_pack_weight_tc: unsupported Cin=%d Cout=%d dtype=%d", Cin, Cout, dtype);
    int units = 9 * (Cin / 32), stages = (units + 1) / 2;
    size_t n = (size_t)stages * Cout * 64;
    int grid = (int)((n + 255) / 256);
    if (dtype == KAD_F16) pack_weight_tc_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>(w_oihw, (__half*)dst, Cin, Cout, stages);
    else pack_weight_tc_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(w_oihw, (__nv_bfloat16*)dst, Cin, Cout, stages);
    KAD_CHECK_LAUNCH("pack_weight_tc_kernel");
    return KAD_OK;
}
