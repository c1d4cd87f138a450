// 3x3 convolution (padding 1, stride 1 or 2) + bias + activation as a TMA-fed tcgen05 implicit GEMM for sm_100a.
//
//   y[b][yo][xo][n] = act( sum_{ky,kx,c} x[b][s*yo+ky-1][s*xo+kx-1][c] * w[n][ky*3+kx][c] + bias[n] )
//
// The op is bound by the L2 -> shared-memory traffic of its operands, not by the tensor pipe, so the design is about
// fetching every byte once per tile:
//  * Activations. For a th x tw tile of output pixels and a 64-channel chunk, ONE tiled TMA load brings the input window
//    (th+2) x (tw+2) (halo included) into shared memory as [window row][window column][64 channels]: one pixel = one
//    128-byte row of the canonical 128-byte-swizzled K-major layout; pixels and channels outside the tensor arrive as
//    zeros, which is the convolution's padding and the K padding at once. All nine taps read that one window: the A
//    operand of tap (ky,kx) is the same buffer started (ky*ww + kx) rows later (ww = window width): the 128-byte swizzle
//    is a function of the shared-memory address alone (TMA writes and the MMA reads agree on it for any 128-byte-
//    aligned start inside a 1024-byte-aligned buffer), so only the descriptor's start address moves, its base-offset
//    field stays 0. Accumulator row m therefore is window position m = ty*ww + tx;
//    the positions with tx >= tw are halo columns whose results are dropped (th*ww <= 128).
//    Stride 2 splits the input by (row, column) parity into four tensor maps, so that the pixels a tap needs are again
//    a dense window: four windows (th+1) x (tw+1) per chunk, tap (ky,kx) reads parity (ky != 1, kx != 1).
//  * Weights [Cout][9][Cin] (3-D tensor map: channel, tap, output channel). When all of them fit beside the windows they
//    are loaded once per CTA and stay resident; otherwise they stream through a ring, one (chunk, tap) slice per
//    stage, and each slice is used for TWO output tiles (two accumulators) before it is released.
// One persistent CTA per SM: warps 0-7 epilogue (TMEM -> bias/activation -> NHWC store, also into a channel slice of
// a wider tensor), warp 8 issues the MMAs, warp 9 loads windows, warp 10 loads weights. Every wait is time-bounded.
#include "kad_common.cuh"
#include "kad_sm100.cuh"

namespace kad {
namespace {
using namespace sm100;

constexpr int C_WSLOTS_MAX = 6, C_BSTAGES_MAX = 8;
constexpr int C_THREADS = 352;
constexpr int C_EPI_WARPS = 8, C_WARP_MMA = 8, C_WARP_WIN = 9, C_WARP_B = 10;

struct ConvMaps {
    CUtensorMap a[4];      // stride 1: a[0]; stride 2: a[py * 2 + px], the input pixels of row parity py and column parity px
    CUtensorMap b;
};

struct ConvParams {
    const float* bias; void* y; int* status;
    int B, Ho, Wo, Cin, N, ldy, act, fmt, stride;
    int th, tw, ww, wh, tiles_y, tiles_x;      // output tile, window width / height
    int nt, n_tiles, chunks;
    int m_tiles, m_super;      // < 2^31 (checked on the host): tile arithmetic stays 32-bit
    int mt;                 // output tiles that share one weight slice (1 or 2)
    int nwin;               // windows per slot: 1 (stride 1) or 4 (stride 2, one per parity)
    int par_bytes;          // bytes of one window (multiple of 1024)
    int win_bytes;          // bytes of one window slot = nwin * par_bytes
    int win_region;         // bytes of all window slots plus the slack the last tap may read past a window
    int wslots, bstages, b_stage_bytes;
    int resident;           // 1: all weight slices live in shared memory for the whole kernel
    int acc_stride, acc_bufs;
};

struct ConvBars {
    uint64_t win_full[C_WSLOTS_MAX], win_empty[C_WSLOTS_MAX];
    uint64_t b_full[C_BSTAGES_MAX], b_empty[C_BSTAGES_MAX];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void creport(int* status, int code, int detail) {
    if (atomicCAS(status, 0, code) == 0) { status[1] = detail; status[2] = blockIdx.x; }
}

struct TileCoord { int img, y0, x0; };
__device__ __forceinline__ TileCoord tile_coord(const ConvParams& p, int mt) {
    const int per = p.tiles_y * p.tiles_x;
    TileCoord c;
    c.img = mt / per;
    const int rem = mt - c.img * per;
    const int tyi = rem / p.tiles_x;
    c.y0 = tyi * p.th; c.x0 = (rem - tyi * p.tiles_x) * p.tw;
    return c;
}

template <typename T>
__global__ void __launch_bounds__(C_THREADS, 1)
conv3x3_tc_kernel(const __grid_constant__ ConvMaps maps, const ConvParams p) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* swin = smem;                                  // [wslots][nwin][window rows][128 B]
    unsigned char* sb = smem + p.win_region;                     // weight slices: ring, or all 9 * chunks of them
    const int b_slices = p.resident ? 9 * p.chunks : p.bstages;
    ConvBars* bars = reinterpret_cast<ConvBars*>(sb + (size_t)b_slices * p.b_stage_bytes);
    volatile int* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nwork = p.m_super * p.n_tiles;

    if (tid == 0) {
        for (int i = 0; i < C_WSLOTS_MAX; ++i) { mbar_init(&bars->win_full[i], 1); mbar_init(&bars->win_empty[i], 1); }
        for (int i = 0; i < C_BSTAGES_MAX; ++i) { mbar_init(&bars->b_full[i], 1); mbar_init(&bars->b_empty[i], 1); }
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

    if (warp < C_EPI_WARPS) {
        const int quad = warp & 3, half = warp >> 2;
        const int r = quad * 32 + lane;                    // accumulator row = window position (r / ww, r % ww)
        const int ty = r / p.ww, tx = r - ty * p.ww;
        const bool in_tile = ty < p.th && tx < p.tw;
        int it = 0;
        for (int work = blockIdx.x; work < nwork; work += gridDim.x, ++it) {
            const int buf = p.acc_bufs == 2 ? (it & 1) : 0;
            const uint32_t par = p.acc_bufs == 2 ? ((it >> 1) & 1) : (it & 1);
            if (!mbar_wait(&bars->acc_full[buf], par, abort_flag)) { creport(p.status, 1, it); break; }
            tc_fence_after();
            const int ms = work / p.n_tiles;
            const int n0 = (work - ms * p.n_tiles) * p.nt;
            const int nchunks = (p.nt + 31) / 32;
            for (int i = 0; i < p.mt; ++i) {
                const int mtile = ms * p.mt + i;
                if (mtile >= p.m_tiles) break;
                const TileCoord tc = tile_coord(p, mtile);
                const int yo = tc.y0 + ty, xo = tc.x0 + tx;
                const bool live = in_tile && yo < p.Ho && xo < p.Wo;
                const long long row = ((long long)tc.img * p.Ho + yo) * p.Wo + xo;
                for (int ch = half; ch < nchunks; ch += 2) {
                    const int c0 = ch * 32;
                    const int nc = min(32, p.nt - c0);
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + (uint32_t)(buf * p.mt * p.acc_stride + i * p.acc_stride + c0) + ((uint32_t)(quad * 32) << 16);
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
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[buf]);
        }
    } else if (warp == C_WARP_MMA) {
        // One thread issues every MMA of the CTA, so this loop is written for the fewest instructions per MMA. All 32
        // lanes run it converged and only the MMA / commit instructions are predicated on lane 0: every value below
        // (ring positions, descriptors) is then provably the same across the warp and stays in uniform registers,
        // which is where tcgen05.mma reads its descriptors from; computed by one diverged lane they would have to be
        // moved there one by one, which costs more than a narrow MMA takes. For the same reason a wait that gives up
        // does not branch out of the loop: it raises the CTA's abort flag, after which every later wait returns at once
        // and the loop runs dry (the results are discarded; the host sees the status word).
        // The descriptors' high words are constants, the low words advance by 32-bit adds, the taps are unrolled.
        const bool leader = lane == 0;
        const uint32_t idesc = instr_desc_f16(p.fmt, p.nt);
        const uint32_t desc_hi = smem_desc_sw128_hi();
        const uint32_t win_lo = smem_desc_sw128_lo(smem_u32(swin)), b_lo_base = smem_desc_sw128_lo(smem_u32(sb));
        const uint32_t win16 = (uint32_t)p.win_bytes >> 4, bst16 = (uint32_t)p.b_stage_bytes >> 4;
        // start row of every tap inside a window, in 16-byte units.
        // stride 1: the window starts at input (y0-1, x0-1), tap (ky,kx) starts ky rows and kx columns in.
        // stride 2: input row 2*yo+ky-1 has parity (ky != 1) and index yo - (ky == 0) among the rows of that parity;
        // the parity windows start at index (y0-1, x0-1), so the tap starts (ky != 0) rows into window (ky != 1, kx != 1).
        uint32_t toff16[9];
#pragma unroll
        for (int tap = 0; tap < 9; ++tap) {
            const int ky = tap / 3, kx = tap % 3;
            toff16[tap] = p.stride == 2
                ? (uint32_t)((((ky != 1) * 2 + (kx != 1)) * p.par_bytes + (((ky != 0) * p.ww + (kx != 0)) << 7)) >> 4)
                : (uint32_t)(((ky * p.ww + kx) << 7) >> 4);
        }
        const int last_nk = (p.Cin - (p.chunks - 1) * 64 + 15) / 16;      // 16-wide K steps of a tap's last channel chunk
        int it = 0;
        int wslot = 0; uint32_t wphase = 0;
        int bslot = 0; uint32_t bphase = 0;
        if (p.resident && !mbar_wait(&bars->b_full[0], 0, abort_flag)) creport(p.status, 5, 0);
        for (int work = blockIdx.x; work < nwork; work += gridDim.x, ++it) {
            const int buf = p.acc_bufs == 2 ? (it & 1) : 0;
            const uint32_t par = p.acc_bufs == 2 ? ((it >> 1) & 1) : (it & 1);
            if (!mbar_wait(&bars->acc_empty[buf], par ^ 1u, abort_flag)) creport(p.status, 2, it);
            tc_fence_after();
            const int ms = work / p.n_tiles;
            const bool two = p.mt == 2 && ms * 2 + 1 < p.m_tiles;
            const uint32_t tacc0 = tmem_base + (uint32_t)(buf * p.mt * p.acc_stride), tacc1 = tacc0 + p.acc_stride;
            uint32_t b_lo = b_lo_base;                  // resident weights: slice (ch, tap) follows slice (ch, tap - 1)
            for (int ch = 0; ch < p.chunks; ++ch) {
                // the windows of this chunk: slots wslot and, for the second tile, the one after it
                if (!mbar_wait(&bars->win_full[wslot], wphase, abort_flag)) creport(p.status, 3, ch);
                const uint32_t wa0 = win_lo + wslot * win16;
                const int ws0 = wslot;
                if (++wslot == p.wslots) { wslot = 0; wphase ^= 1u; }
                uint32_t wa1 = 0; int ws1 = 0;
                if (two) {
                    if (!mbar_wait(&bars->win_full[wslot], wphase, abort_flag)) creport(p.status, 3, ch);
                    wa1 = win_lo + wslot * win16; ws1 = wslot;
                    if (++wslot == p.wslots) { wslot = 0; wphase ^= 1u; }
                }
                tc_fence_after();
                const int nk = (ch == p.chunks - 1) ? last_nk : 4;
                uint32_t first = ch ? 1u : 0u;          // the very first MMA of a tile overwrites the accumulator
#pragma unroll
                for (int tap = 0; tap < 9; ++tap) {
                    if (!p.resident) {
                        if (!mbar_wait(&bars->b_full[bslot], bphase, abort_flag)) creport(p.status, 4, tap);
                        tc_fence_after();
                        b_lo = b_lo_base + bslot * bst16;
                    }
                    const uint32_t a0 = wa0 + toff16[tap], a1 = wa1 + toff16[tap];
                    if (nk == 4) {
                        if (leader) {
                            umma_f16_lohi(tacc0, a0, b_lo, desc_hi, idesc, first);
                            umma_f16_lohi(tacc0, a0 + 2, b_lo + 2, desc_hi, idesc, 1u);
                            umma_f16_lohi(tacc0, a0 + 4, b_lo + 4, desc_hi, idesc, 1u);
                            umma_f16_lohi(tacc0, a0 + 6, b_lo + 6, desc_hi, idesc, 1u);
                        }
                        if (two && leader) {
                            umma_f16_lohi(tacc1, a1, b_lo, desc_hi, idesc, first);
                            umma_f16_lohi(tacc1, a1 + 2, b_lo + 2, desc_hi, idesc, 1u);
                            umma_f16_lohi(tacc1, a1 + 4, b_lo + 4, desc_hi, idesc, 1u);
                            umma_f16_lohi(tacc1, a1 + 6, b_lo + 6, desc_hi, idesc, 1u);
                        }
                    } else {
                        for (int k = 0; k < nk; ++k)
                            if (leader) umma_f16_lohi(tacc0, a0 + 2 * k, b_lo + 2 * k, desc_hi, idesc, k ? 1u : first);
                        if (two)
                            for (int k = 0; k < nk; ++k)
                                if (leader) umma_f16_lohi(tacc1, a1 + 2 * k, b_lo + 2 * k, desc_hi, idesc, k ? 1u : first);
                    }
                    first = 1u;
                    if (p.resident) b_lo += bst16;
                    else {
                        if (leader) umma_commit(&bars->b_empty[bslot]);
                        if (++bslot == p.bstages) { bslot = 0; bphase ^= 1u; }
                    }
                }
                if (leader) {
                    umma_commit(&bars->win_empty[ws0]);
                    if (two) umma_commit(&bars->win_empty[ws1]);
                    if (ch == p.chunks - 1) umma_commit(&bars->acc_full[buf]);
                }
            }
        }
        __syncwarp();
    }
    else if (warp == C_WARP_WIN) {
        if (lane == 0) {
            for (int i = 0; i < p.nwin; ++i) tma_prefetch_desc(&maps.a[i]);
            long long issued = 0;
            int ws = 0; uint32_t wp = 0;
            bool ok = true;
            const uint32_t tx_bytes = (uint32_t)(p.nwin * p.wh * p.ww * 128);
            for (int work = blockIdx.x; work < nwork && ok; work += gridDim.x) {
                const int ms = work / p.n_tiles;
                const int mt_eff = min(p.mt, p.m_tiles - ms * p.mt);
                for (int ch = 0; ch < p.chunks && ok; ++ch) {
                    for (int i = 0; i < mt_eff; ++i, ++issued) {
                        if (!mbar_wait(&bars->win_empty[ws], wp ^ 1u, abort_flag)) { creport(p.status, 6, ch); ok = false; break; }
                        const TileCoord tc = tile_coord(p, ms * p.mt + i);
                        mbar_arrive_expect_tx(&bars->win_full[ws], tx_bytes);
                        for (int q = 0; q < p.nwin; ++q)
                            tma_load_4d(swin + (size_t)ws * p.win_bytes + (size_t)q * p.par_bytes, &maps.a[q], ch * 64, tc.x0 - 1, tc.y0 - 1, tc.img,
                                        &bars->win_full[ws]);
                        if (++ws == p.wslots) { ws = 0; wp ^= 1u; }
                    }
                }
            }
            if (!ok || *abort_flag) {
                // the copies already issued must land before the block may exit
                for (int i = 0; i < p.wslots && i < issued; ++i) {
                    const long long j = issued - 1 - i;
                    mbar_wait(&bars->win_full[j % p.wslots], (uint32_t)((j / p.wslots) & 1), abort_flag);
                }
            }
        }
    } else if (warp == C_WARP_B) {
        if (lane == 0) {
            tma_prefetch_desc(&maps.b);
            if (p.resident) {
                mbar_arrive_expect_tx(&bars->b_full[0], (uint32_t)(9 * p.chunks * p.nt * 128));
                for (int ch = 0; ch < p.chunks; ++ch)
                    for (int tap = 0; tap < 9; ++tap)
                        tma_load_3d(sb + (size_t)(ch * 9 + tap) * p.b_stage_bytes, &maps.b, ch * 64, tap, 0, &bars->b_full[0]);
                // the block's last barrier below is reached only after the MMA warp has seen these copies land (or
                // after the bounded wait for them has given up), so nothing is in flight when the block exits
            } else {
                long long issued = 0;
                int bs = 0; uint32_t bp = 0;
                bool ok = true;
                const uint32_t tx_bytes = (uint32_t)(p.nt * 128);
                for (int work = blockIdx.x; work < nwork && ok; work += gridDim.x) {
                    const int ms = work / p.n_tiles;
                    const int n0 = (work - ms * p.n_tiles) * p.nt;
                    for (int ch = 0; ch < p.chunks && ok; ++ch)
                        for (int tap = 0; tap < 9; ++tap, ++issued) {
                            if (!mbar_wait(&bars->b_empty[bs], bp ^ 1u, abort_flag)) { creport(p.status, 7, tap); ok = false; break; }
                            mbar_arrive_expect_tx(&bars->b_full[bs], tx_bytes);
                            tma_load_3d(sb + (size_t)bs * p.b_stage_bytes, &maps.b, ch * 64, tap, n0, &bars->b_full[bs]);
                            if (++bs == p.bstages) { bs = 0; bp ^= 1u; }
                        }
                }
                if (!ok || *abort_flag) {
                    for (int i = 0; i < p.bstages && i < issued; ++i) {
                        const long long j = issued - 1 - i;
                        mbar_wait(&bars->b_full[j % p.bstages], (uint32_t)((j / p.bstages) & 1), abort_flag);
                    }
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

namespace {
inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Tiling and shared-memory plan of one problem; returns false if nothing fits (does not happen for supported shapes).
bool plan_conv(ConvParams& p, int sms) {
    const int halo = p.stride == 1 ? 2 : 1;
    p.nwin = p.stride == 1 ? 1 : 4;
    const int slot_cap = p.stride == 1 ? 40 * 1024 : 56 * 1024;
    // output tile th x tw: th * (tw + halo) accumulator rows <= 128 and a window slot within its cap; the fewest tiles
    // win, then the smallest window
    long long best_tiles = -1; int best_bytes = 0;
    for (int th = 1; th <= 128 && th <= p.Ho; ++th)
        for (int tw = 1; tw <= p.Wo && th * (tw + halo) <= 128; ++tw) {
            const int ww = tw + halo, wh = th + halo;
            const int par = round_up(wh * ww * 128, 1024);
            if (p.nwin * par > slot_cap) continue;
            const long long t = (long long)((p.Ho + th - 1) / th) * ((p.Wo + tw - 1) / tw);
            if (best_tiles < 0 || t < best_tiles || (t == best_tiles && par < best_bytes)) {
                best_tiles = t; best_bytes = par; p.th = th; p.tw = tw;
            }
        }
    if (best_tiles < 0) return false;
    p.ww = p.tw + halo; p.wh = p.th + halo;
    p.par_bytes = round_up(p.wh * p.ww * 128, 1024);
    p.win_bytes = p.nwin * p.par_bytes;
    p.tiles_y = (p.Ho + p.th - 1) / p.th; p.tiles_x = (p.Wo + p.tw - 1) / p.tw;
    const long long mtl = (long long)p.B * p.tiles_y * p.tiles_x;
    if (mtl * ((p.N + 255) / 256) >= (1ll << 31)) return false;
    p.m_tiles = (int)mtl;
    p.n_tiles = (p.N + 255) / 256;
    p.nt = round_up((p.N + p.n_tiles - 1) / p.n_tiles, 16);
    p.chunks = (p.Cin + 63) / 64;
    p.b_stage_bytes = p.nt * 128;
    p.acc_stride = round_up(p.nt, 32);
    // an MMA always reads 128 rows from its start row, and the last tap starts 2*ww+2 rows into the window
    const int reach = (128 + 2 * p.ww + 2) * 128;
    const int slack = reach > p.par_bytes ? round_up(reach - p.par_bytes, 1024) : 0;
    const int fixed = (int)sizeof(ConvBars) + p.n_tiles * p.nt * 4 + 32 + 1024;
    const int avail = 226 * 1024 - fixed - slack;
    const int wbytes = 9 * p.chunks * p.b_stage_bytes;
    p.resident = 0; p.mt = 1; p.bstages = 0; p.wslots = 0;
    if (p.n_tiles == 1 && wbytes + 2 * p.win_bytes <= avail) {
        p.resident = 1;
        p.wslots = (avail - wbytes) / p.win_bytes;
    } else {
        // streamed weights: two tiles per weight slice when there is enough work and room for their windows
        const int want_mt = p.m_tiles >= 2 * sms ? 2 : 1;
        for (int mt = want_mt; mt >= 1 && !p.wslots; --mt)
            for (int bst = 4; bst >= 2 && !p.wslots; --bst) {
                const int ws = (avail - bst * p.b_stage_bytes) / p.win_bytes;
                if (ws >= 2 * mt || (bst == 2 && ws >= mt)) { p.mt = mt; p.bstages = bst; p.wslots = ws; }
            }
        if (!p.wslots) return false;
    }
    if (p.wslots > C_WSLOTS_MAX) p.wslots = C_WSLOTS_MAX;
    if (p.wslots > 2 * p.mt + 2) p.wslots = 2 * p.mt + 2;
    p.win_region = p.wslots * p.win_bytes + slack;
    p.acc_bufs = 2 * p.mt * p.acc_stride <= 512 ? 2 : 1;
    p.m_super = (p.m_tiles + p.mt - 1) / p.mt;
    return true;
}
}  // namespace

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
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

    ConvParams p{};
    p.bias = bias; p.y = y; p.status = status;
    p.B = B; p.Cin = Cin; p.N = Cout; p.ldy = ldy; p.act = act; p.stride = stride;
    p.Ho = (H - 1) / stride + 1; p.Wo = (W - 1) / stride + 1;          // kernel 3, padding 1
    p.fmt = dtype == KAD_BF16 ? 1 : 0;
    if (!plan_conv(p, sms)) return fail(KAD_ERR_UNSUPPORTED, "kad_conv3x3_bias_act: no shared-memory plan for Cin=%d Cout=%d", Cin, Cout);

    ConvMaps maps;
    CUtensorMapDataType dt = dtype == KAD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    for (int q = 0; q < p.nwin; ++q) {
        const int py = q >> 1, px = q & 1;
        // the pixels of row parity py and column parity px (stride 2), or all pixels (stride 1)
        const int Hq = stride == 2 ? (H - py + 1) / 2 : H, Wq = stride == 2 ? (W - px + 1) / 2 : W;
        const char* base = reinterpret_cast<const char*>(x) + (stride == 2 ? ((size_t)py * W + px) * ldx * 2 : 0);
        cuuint64_t dims[4] = {(cuuint64_t)Cin, (cuuint64_t)Wq, (cuuint64_t)Hq, (cuuint64_t)B};
        cuuint64_t strides[3] = {(cuuint64_t)stride * ldx * 2, (cuuint64_t)stride * W * ldx * 2, (cuuint64_t)H * W * ldx * 2};
        cuuint32_t box[4] = {64, (cuuint32_t)p.ww, (cuuint32_t)p.wh, 1};
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
    const int b_slices = p.resident ? 9 * p.chunks : p.bstages;
    const size_t smem = (size_t)p.win_region + (size_t)b_slices * p.b_stage_bytes + sizeof(ConvBars) + (size_t)p.n_tiles * p.nt * 4 + 32 + 1024;
    const int nwork = p.m_super * p.n_tiles;
    const int grid = nwork < sms ? nwork : sms;
    cudaError_t e;
    if (dtype == KAD_F16) {
        auto kern = conv3x3_tc_kernel<__half>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "conv3x3 smem attribute (%zu bytes): %s", smem, cudaGetErrorString(e));
        kern<<<grid, C_THREADS, smem, (cudaStream_t)stream>>>(maps, p);
    } else {
        auto kern = conv3x3_tc_kernel<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "conv3x3 smem attribute (%zu bytes): %s", smem, cudaGetErrorString(e));
        kern<<<grid, C_THREADS, smem, (cudaStream_t)stream>>>(maps, p);
    }
    KAD_CHECK_LAUNCH("conv3x3_tc_kernel");
    return KAD_OK;
}


