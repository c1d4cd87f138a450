// Deformable 3x3 convolution for SMALL channel counts (the detector's DSCs have 10-44 channels) on the warp-level
// tensor-core instruction (mma.sync m16n8k16, fp16/bf16 operands, fp32 accumulators), NHWC.
//
// Why not the tcgen05 implicit GEMM: with K = 9 taps x 10..44 channels and N <= 64 the contraction is tiny; what costs
// is the bilinear gather. So the A operand is never staged as a matrix: the four lanes that share an accumulator row
// gather four channels each (one 8-byte load per corner) straight into the A-fragment registers. The bilinear
// interpolation itself is folded into the contraction: a sample is sum_corner w_corner * x[corner], so every corner
// contributes one MMA with A = w_corner * x[corner] (one packed multiply per register) against the same weight
// fragment; products are rounded to the storage type, the sum over corners, taps and channels is fp32.
//
// Blocks are persistent (two per SM for the narrow variants) and walk over (image, group of 256 consecutive pixels);
// a warp owns 32 pixels of the group (two 16-row MMA tiles). The image rows a group can reach (its own rows, one row of
// 3x3 halo, a margin for the learned offsets) are one CONTIGUOUS range of the NHWC tensor; it is copied to shared
// memory with 16-byte cp.async, so HBM sees one coalesced pass over x and the gathers are shared-memory loads with
// 32-bit addresses. Lane l computes the sampling geometry of pixel l, one kernel row (3 taps) at a time, into a
// warp-private table: per corner the shared-memory address of the pixel (the address of a block of zeros when the
// corner leaves the image) and the mask-scaled weight. The gathering lanes then run straight-line code: address +
// channel offset, one load, multiply, MMA. A tap in which some lane's sample leaves the staged rows (a warp vote)
// takes a slower variant of the same code that reads those corners from global memory.
// Results leave through shared memory as well, so that a warp writes its 32 pixels as one contiguous run.
//
// Modes:  plain   offset == NULL: ordinary zero-padded 3x3 convolution (the offset convolution, c -> 18)
//         deform  offsets and modulation mask read from global memory
//         fused   the offset convolution runs first on the same pixels and its 18 outputs go through shared memory
//                 straight into the sampling geometry: the offset tensor never exists in global memory.
//         inline  fused, and the LCSA modulation mask (kad_conv.py:24-39,:65) is evaluated by the lane that owns the pixel
//                 from the row means and the per-column terms of the separable 1x11 stage (a few KB per image, prepared
//                 by the pyramid kernel): the mask tensor (36 bytes per pixel, written and read back) never exists either.
#include "kad_mma.cuh"

namespace kad {
namespace {

constexpr int MMA_WARPS = 8;
constexpr int OFF_PITCH = 19;           // floats per pixel of the staged offsets (18, padded against bank conflicts)
constexpr int NT_OFF = 3;               // n-tiles of the offset convolution (18 outputs -> 24)

struct MmaParams {
    const void* x; const void* offset; const void* mask;
    const float* Wt;                    // [9][Cin][Cout] fp32
    const float* Woff;                  // [9][Cin][18] fp32 (fused mode)
    const float* boff;                  // [18] (fused mode)
    const float* scale; const float* shift; const float* post;
    void* y; float* gap_partial;
    int H, W, Cin, Cout, KC, align;
    int offset_f32, mask_f32, y_f32, act;
    int B, win_margin;                  // win_margin: rows staged above / below the 3x3 halo for the learned offsets
    // inline mode: LCSA operands. rowmean [B][H][Cin] (means over x), A [B][W][Cp], Sm [W][Cp] (Cp = Cin rounded up to 4),
    // w2 [Cin][11], b2 [Cin], w3 [9][Cin], b3 [9]
    const float* l_rowmean; const float* l_A; const float* l_Sm; const float* l_w2; const float* l_b2; const float* l_w3; const float* l_b3;
    int Cp, rm_rows;                    // rm_rows: image rows a group of 256 pixels can span, + 10 for the 11x1 window
    int stage_cols;                     // 1: the image's A rows and Sm are staged in shared memory (they fit); 0: read through L2
};

constexpr int SCRATCH_PER_WARP = 4224;  // sampling table (3 taps x 32 pixels x 32 bytes), later the warp's output tile (+ 16 bytes of shift)
constexpr int ZERO_BYTES = 160;         // block of zeros in shared memory that out-of-image corners point at
constexpr uint32_t OUTSIDE = 0x80000000u;   // table address flag: the corner is not staged; low bits = image element offset

// Weight fragments for mma.sync: lane (g = lane / 4, t = lane % 4) of n-tile nt holds output channel nt*8 + g and four
// input channels (the K order inside a 16-chunk is permuted so that a lane's four A values are four CONSECUTIVE
// channels: logical k = 2t, 2t+1, 2t+8, 2t+9  <->  slot 0..3 = channel first + 0..3, first = lane_first_channel()).
template <typename T>
__device__ __forceinline__ void stage_weights(uint2* dst, const float* __restrict__ Wt, int Cin, int Cout, int KC, int NT, int tid) {
    const int total = 9 * KC * NT * 32;
    for (int e = tid; e < total; e += MMA_THREADS) {
        const int lane = e & 31, f = e >> 5, nt = f % NT, kc = (f / NT) % KC, k = f / (NT * KC);
        const int n = nt * 8 + (lane >> 2), t = lane & 3, ch = kc * 16 + 4 * t;
        const int first = lane_first_channel(kc, t, Cin);
        float w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = first + j;
            w[j] = (n < Cout && c >= ch && c < Cin) ? Wt[((size_t)k * Cin + c) * Cout + n] : 0.f;
        }
        dst[e] = make_uint2(pack2<T>(w[0], w[1]), pack2<T>(w[2], w[3]));
    }
}

// Ordinary 3x3 convolution of this lane's four accumulator rows over all taps and chunks, out of the staged rows.
// so[j] = shared-memory address of row j's pixel, vm[j] = which of its 9 neighbours lie inside the image.
// KCT: the number of 16-channel chunks when it is known at compile time (1 or 2: the detector's widths), 0 = use KCr.
template <typename T, int NTP, int ALIGN, int KCT>
__device__ __forceinline__ void plain_pass(float (&acc)[2][NTP][4], const unsigned char* smem, const uint32_t (&so)[4], const uint32_t (&vm)[4],
                                           uint32_t zoff, const uint2* __restrict__ Bs, int KCr, int Cin, int W, int lane) {
    const int KC = KCT ? KCT : KCr;
    const int t = lane & 3;
#pragma unroll 3
    for (int k = 0; k < 9; ++k) {
        const int step = ((k / 3 - 1) * W + (k % 3 - 1)) * Cin * 2;
        uint32_t q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = ((vm[j] >> k) & 1u) ? so[j] + step : zoff;
#pragma unroll (KCT ? KCT : 1)
        for (int kc = 0; kc < KC; ++kc) {
            const uint32_t coff = 2 * lane_first_channel(kc, t, Cin);
            uint2 bf[NTP];
#pragma unroll
            for (int nt = 0; nt < NTP; ++nt) bf[nt] = Bs[((k * KC + kc) * NTP + nt) * 32 + lane];
            uint2 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = lds8<ALIGN>(smem, q[j] + coff);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTP; ++nt) mma16816<T>(acc[mt][nt], v[2 * mt].x, v[2 * mt + 1].x, v[2 * mt].y, v[2 * mt + 1].y, bf[nt]);
        }
    }
}

// One tap of the deformable pass for one 16-row tile: A = corner weight * gathered channels, four corners, all chunks.
// SLOW: some address in the warp carries the OUTSIDE flag and is read from global memory instead.
template <typename T, int NT, int ALIGN, bool SLOW, int KCT>
__device__ __forceinline__ void deform_tap(float (&acc)[NT][4], const unsigned char* smem, const unsigned char* gimg, const uint4* tw, const uint4* ta,
                                           int row0, const uint2* __restrict__ Bs, int k, int KCr, int Cin, int lane) {
    const int KC = KCT ? KCT : KCr;
    const int t = lane & 3;
    uint32_t w[2][4], a[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint4 wq = tw[row0 + 8 * h], aq = ta[row0 + 8 * h];
        w[h][0] = wq.x; w[h][1] = wq.y; w[h][2] = wq.z; w[h][3] = wq.w;
        a[h][0] = aq.x; a[h][1] = aq.y; a[h][2] = aq.z; a[h][3] = aq.w;
    }
#pragma unroll (KCT ? KCT : 1)
    for (int kc = 0; kc < KC; ++kc) {
        const uint32_t coff = 2 * lane_first_channel(kc, t, Cin);
        uint2 bf[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) bf[nt] = Bs[((k * KC + kc) * NT + nt) * 32 + lane];
        uint2 v[2][4];
#pragma unroll
        for (int cr = 0; cr < 4; ++cr)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (SLOW && (a[h][cr] & OUTSIDE)) v[h][cr] = ldg8<ALIGN>(gimg + 2 * (size_t)(a[h][cr] & ~OUTSIDE) + coff);
                else v[h][cr] = lds8<ALIGN>(smem, a[h][cr] + coff);
            }
#pragma unroll
        for (int cr = 0; cr < 4; ++cr) {
            const uint32_t a0 = mul2<T>(v[0][cr].x, w[0][cr]), a2 = mul2<T>(v[0][cr].y, w[0][cr]);
            const uint32_t a1 = mul2<T>(v[1][cr].x, w[1][cr]), a3 = mul2<T>(v[1][cr].y, w[1][cr]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma16816<T>(acc[nt], a0, a1, a2, a3, bf[nt]);
        }
    }
}

// LCSA modulation mask of one pixel (column x of image row h), the arithmetic of lcsa_mask_flat_kernel in the same order:
//   h1(r, c) = relu(rowmean[r][c] * Sm[x][c] + A[x][c])        (1x11 depthwise + BatchNorm + ReLU, separated)
//   v(c)     = b2[c] + sum_k w2[c][k] * h1(h + k - 5, c)       (11x1 depthwise, zero padding: rows outside contribute 0)
//   mask[j]  = sigmoid(b3[j] + sum_c w3[j][c] * v(c))
// rm: staged row means, row (h - 5) first, Cp floats per row; sw2 / sw3: [Cp][12] (slot 11 of sw2 = b2); valid: bit k set
// when row h + k - 5 lies inside the image (BORDER = false: the caller knows all 11 rows do).
template <bool BORDER>
__device__ __forceinline__ void lcsa_mask_pixel(float (&mk)[9], const float* A, const float* Sm, const float* rm,
                                                const float* sw2, const float* sw3, const float* __restrict__ b3, int Cp, uint32_t valid) {
    float logit[9];
#pragma unroll
    for (int j = 0; j < 9; ++j) logit[j] = __ldg(b3 + j);
    const float4* A4 = reinterpret_cast<const float4*>(A);
    const float4* S4 = reinterpret_cast<const float4*>(Sm);
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
            const float4 u0 = w24[3 * c], u1 = w24[3 * c + 1], u2 = w24[3 * c + 2];
            const float uk[11] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w, u2.x, u2.y, u2.z};
            float v = u2.w;           // bias of the 11x1 convolution (0 for a padding channel, whose weights are 0 as well)
            const float* r = rm + c;
#pragma unroll
            for (int k = 0; k < 11; ++k) {
                float tv = fmaxf(fmaf(r[k * Cp], s, a), 0.f);
                if (BORDER && !((valid >> k) & 1u)) tv = 0.f;
                v = fmaf(uk[k], tv, v);
            }
            const float4 q0 = w34[3 * c], q1 = w34[3 * c + 1], q2 = w34[3 * c + 2];
            logit[0] = fmaf(q0.x, v, logit[0]); logit[1] = fmaf(q0.y, v, logit[1]); logit[2] = fmaf(q0.z, v, logit[2]);
            logit[3] = fmaf(q0.w, v, logit[3]); logit[4] = fmaf(q1.x, v, logit[4]); logit[5] = fmaf(q1.y, v, logit[5]);
            logit[6] = fmaf(q1.z, v, logit[6]); logit[7] = fmaf(q1.w, v, logit[7]); logit[8] = fmaf(q2.x, v, logit[8]);
        }
    }
#pragma unroll
    for (int j = 0; j < 9; ++j) mk[j] = sigmoidf_(logit[j]);
}

template <typename T, int NT, int MODE, int ALIGN, int KCT>      // MODE 0 plain, 1 deform, 2 fused, 3 fused + inline LCSA mask
__global__ void __launch_bounds__(MMA_THREADS, NT <= 4 ? 2 : 1)
dsc_mma_kernel(const MmaParams p) {
    constexpr int COP = NT * 8;
    extern __shared__ __align__(16) unsigned char smem_mma[];
    const int KC = KCT ? KCT : p.KC;
    uint2* Bs = reinterpret_cast<uint2*>(smem_mma);                                   // [9][KC][NT][32]
    constexpr bool FUSED = MODE >= 2, INLINE = MODE == 3;
    uint2* Bo = Bs + 9 * KC * NT * 32;                                                // [9][KC][3][32]   (fused)
    unsigned char* cur = reinterpret_cast<unsigned char*>(Bo + (FUSED ? 9 * KC * NT_OFF * 32 : 0));
    unsigned char* scratch = cur; cur += MMA_WARPS * SCRATCH_PER_WARP;
    float* ep = reinterpret_cast<float*>(cur); cur += 3 * COP * 4;                    // scale | shift | post
    float* red = reinterpret_cast<float*>(cur); cur += MMA_WARPS * COP * 4;
    float* offs = reinterpret_cast<float*>(cur); cur += (FUSED ? MMA_WARPS * 32 * OFF_PITCH * 4 : 0);
    float* boffs = reinterpret_cast<float*>(cur); cur += (FUSED ? 32 * 4 : 0);        // [24] (fused)
    float* sw2 = reinterpret_cast<float*>(cur); cur += (INLINE ? p.Cp * 48 : 0);      // [Cp][12] 11x1 taps, slot 11 = bias (inline)
    float* sw3 = reinterpret_cast<float*>(cur); cur += (INLINE ? p.Cp * 48 : 0);      // [Cp][12] 1x1 weights of the 9 mask outputs
    float* rms = reinterpret_cast<float*>(cur); cur += (INLINE ? p.rm_rows * p.Cp * 4 : 0);   // [rm_rows][Cp] row means of the group's rows
    float* As = reinterpret_cast<float*>(cur); cur += ((INLINE && p.stage_cols) ? p.W * p.Cp * 4 : 0);     // [W][Cp] column terms of the current image
    float* Sms = reinterpret_cast<float*>(cur); cur += ((INLINE && p.stage_cols) ? p.W * p.Cp * 4 : 0);    // [W][Cp] (the same for every image)
    const uint32_t zoff = static_cast<uint32_t>(cur - smem_mma); cur += ZERO_BYTES;   // the block of zeros
    const uint32_t wdata = static_cast<uint32_t>(cur - smem_mma) + 16;                // staged rows start here (16 bytes of slack in front)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int H = p.H, W = p.W, HW = H * W, Cin = p.Cin, Cout = p.Cout;
    const int gpi = (HW + MMA_THREADS - 1) / MMA_THREADS, total = gpi * p.B;      // groups per image, groups in all

    uint4* my_w = reinterpret_cast<uint4*>(scratch + warp * SCRATCH_PER_WARP);    // [3][32] corner weights, each a duplicated pair
    uint4* my_a = my_w + 96;                                                          // [3][32] corner addresses
    unsigned char* my_tile = scratch + warp * SCRATCH_PER_WARP;                       // output tile (after the taps are done)
    float* my_offs = offs + warp * 32 * OFF_PITCH;
    const float relu_floor = p.act == KAD_ACT_RELU ? 0.f : -INFINITY;

    bool first = true;
    for (int gi = blockIdx.x; gi < total; gi += gridDim.x) {
        const int b = gi / gpi, grp = gi - b * gpi, base = grp * MMA_THREADS;
        const unsigned char* gimg = reinterpret_cast<const unsigned char*>(p.x) + (size_t)b * HW * Cin * 2;
        // ---- stage the rows this group can reach -------------------------------------------------------------
        __syncthreads();                                       // every warp is done with the previous rows, tiles and sums
        const int last = min(HW, base + MMA_THREADS) - 1;
        const int wy0 = max(0, base / W - 1 - p.win_margin), wy1 = min(H - 1, last / W + 1 + p.win_margin);
        const int e_lo = wy0 * W * Cin, e_hi = (wy1 + 1) * W * Cin;                  // staged image elements [e_lo, e_hi)
        const uintptr_t a_lo = reinterpret_cast<uintptr_t>(gimg) + 2 * (size_t)e_lo, a16 = a_lo & ~uintptr_t(15);
        const uintptr_t a_hi = reinterpret_cast<uintptr_t>(gimg) + 2 * (size_t)e_hi;
        if (INLINE) {
            // first copy group: row means of the rows this group's 11x1 windows reach (0 outside the image) and the image's column terms
            const int r_lo = base / W, nrm = last / W - r_lo + 11;
            for (int e = tid; e < nrm * p.Cp; e += MMA_THREADS) {
                const int j = e / p.Cp, c = e - j * p.Cp, hh = r_lo - 5 + j;
                if (hh >= 0 && hh < H && c < Cin) cp_async4(rms + e, p.l_rowmean + ((size_t)b * H + hh) * Cin + c);
                else rms[e] = 0.f;
            }
            if (p.stage_cols) {
                const float* Ag = p.l_A + (size_t)b * W * p.Cp;
                for (int i = tid; i < (W * p.Cp) >> 2; i += MMA_THREADS) cp_async16(As + 4 * i, Ag + 4 * i);
            }
            cp_async_commit();
        }
        {
            const int nbytes = static_cast<int>(a_hi - a16), nvec = nbytes >> 4, ntail = (nbytes & 15) >> 1;
            unsigned char* dst = smem_mma + wdata;
            for (int i = tid; i < nvec; i += MMA_THREADS) cp_async16(dst + 16 * i, reinterpret_cast<const void*>(a16 + 16 * (size_t)i));
            if (tid < ntail)
                *reinterpret_cast<uint16_t*>(dst + 16 * nvec + 2 * tid) = *reinterpret_cast<const uint16_t*>(a16 + 16 * (size_t)nvec + 2 * tid);
            if (INLINE) cp_async_commit();                     // second copy group: the image rows
        }
        // shared-memory address of image element e: sel0 + 2*e
        const int sel0 = static_cast<int>(wdata) - static_cast<int>(static_cast<ptrdiff_t>(a16) - static_cast<ptrdiff_t>(reinterpret_cast<uintptr_t>(gimg)));
        if (first) {
            stage_weights<T>(Bs, p.Wt, Cin, Cout, KC, NT, tid);
            if (FUSED) {
                stage_weights<T>(Bo, p.Woff, Cin, 18, KC, NT_OFF, tid);
                if (tid < 24) boffs[tid] = (tid < 18 && p.boff) ? p.boff[tid] : 0.f;
            }
            if (INLINE) {
                for (int e = tid; e < 12 * p.Cp; e += MMA_THREADS) {
                    const int c = e / 12, k = e - c * 12;
                    sw3[e] = (k < 9 && c < Cin) ? p.l_w3[k * Cin + c] : 0.f;
                    sw2[e] = c < Cin ? (k < 11 ? p.l_w2[c * 11 + k] : p.l_b2[c]) : 0.f;
                }
                if (p.stage_cols) for (int e = tid; e < W * p.Cp; e += MMA_THREADS) Sms[e] = p.l_Sm[e];
            }
            for (int e = tid; e < COP; e += MMA_THREADS) {
                const bool on = e < Cout;
                ep[e] = (on && p.scale) ? p.scale[e] : 1.f;
                ep[COP + e] = (on && p.shift) ? p.shift[e] : 0.f;
                ep[2 * COP + e] = (on && p.post) ? p.post[e] : 1.f;
            }
            if (tid < ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(smem_mma + zoff)[tid] = 0u;
            first = false;
        }
        // lane l describes pixel wbase + l; its modulation mask is fetched while the copy is in flight
        const int wbase = base + warp * 32;
        const int mypix = wbase + lane;
        const bool mylive = mypix < HW;
        const int mpy = mypix / W, mpx = mypix - mpy * W;
        const size_t gp = (size_t)b * HW + mypix;
        float mk[9];
        if (INLINE) {
            // the LCSA operands have landed (the image rows may still be in flight): every lane evaluates its pixel's mask
            const int r_lo = base / W;
            cp_async_wait_but_one();
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 9; ++k) mk[k] = 1.f;
            uint32_t valid = 0x7ffu;
            if (mylive) {
                valid = 0;
#pragma unroll
                for (int k = 0; k < 11; ++k) valid |= (uint32_t)(mpy + k - 5 >= 0 && mpy + k - 5 < H) << k;
            }
            const bool border = __any_sync(0xffffffffu, valid != 0x7ffu);
            if (mylive) {
                const float* Ap = p.stage_cols ? As + mpx * p.Cp : p.l_A + ((size_t)b * W + mpx) * p.Cp;
                const float* Sp = p.stage_cols ? Sms + mpx * p.Cp : p.l_Sm + (size_t)mpx * p.Cp;
                const float* rmp = rms + (mpy - r_lo) * p.Cp;
                if (border) lcsa_mask_pixel<true>(mk, Ap, Sp, rmp, sw2, sw3, p.l_b3, p.Cp, valid);
                else lcsa_mask_pixel<false>(mk, Ap, Sp, rmp, sw2, sw3, p.l_b3, p.Cp, valid);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 9; ++k) mk[k] = (MODE != 0 && mylive && p.mask) ? load_mixed<T>(p.mask, gp * 9 + k, p.mask_f32) : 1.f;
        }
        uint32_t myvm = 0;                                     // which 3x3 neighbours of my pixel are inside the image
        if (mylive) {
#pragma unroll
            for (int k = 0; k < 9; ++k) {
                const int yy = mpy + k / 3 - 1, xx = mpx + k % 3 - 1;
                if (yy >= 0 && yy < H && xx >= 0 && xx < W) myvm |= 1u << k;
            }
        }
        cp_async_wait_all();
        __syncthreads();

        float psum[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) psum[nt][0] = psum[nt][1] = 0.f;
        if (wbase < HW) {
            // the four accumulator rows of this lane: j = mt*2 + half -> pixel wbase + mt*16 + g + 8*half
            uint32_t so[4], vm[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = (j >> 1) * 16 + g + 8 * (j & 1);
                vm[j] = __shfl_sync(0xffffffffu, myvm, r);
                so[j] = static_cast<uint32_t>(sel0 + 2 * (wbase + r) * Cin);
            }
            float acc[2][NT][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

            if (MODE == 0) {
                plain_pass<T, NT, ALIGN, KCT>(acc, smem_mma, so, vm, zoff, Bs, KC, Cin, W, lane);
            } else {
                if (FUSED) {
                    // offset convolution of the warp's 32 pixels -> shared memory [32][18]
                    float oacc[2][NT_OFF][4];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int nt = 0; nt < NT_OFF; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) oacc[mt][nt][i] = 0.f;
                    plain_pass<T, NT_OFF, ALIGN, KCT>(oacc, smem_mma, so, vm, zoff, Bo, KC, Cin, W, lane);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int nt = 0; nt < NT_OFF; ++nt) {
                            const int co = nt * 8 + 2 * t, row = (j >> 1) * 16 + g + 8 * (j & 1);
                            if (co < 18) {
                                my_offs[row * OFF_PITCH + co] = oacc[j >> 1][nt][2 * (j & 1)] + boffs[co];
                                my_offs[row * OFF_PITCH + co + 1] = oacc[j >> 1][nt][2 * (j & 1) + 1] + boffs[co + 1];
                            }
                        }
                }
#pragma unroll (KCT ? 3 : 1)
                for (int r = 0; r < 3; ++r) {
                    __syncwarp();                              // readers of the previous row's table are done; offsets are visible
                    uint32_t slow = 0;                         // bit kk: some lane's sample of tap kk leaves the staged rows
#pragma unroll
                    for (int kk = 0; kk < 3; ++kk) {
                        const int k = 3 * r + kk;
                        uint4 wq = make_uint4(0u, 0u, 0u, 0u), aq = make_uint4(zoff, zoff, zoff, zoff);
                        bool out = false;
                        if (mylive) {
                            float dy, dx;
                            if (FUSED) { dy = my_offs[lane * OFF_PITCH + 2 * k]; dx = my_offs[lane * OFF_PITCH + 2 * k + 1]; }
                            else { dy = load_mixed<T>(p.offset, gp * 18 + 2 * k, p.offset_f32); dx = load_mixed<T>(p.offset, gp * 18 + 2 * k + 1, p.offset_f32); }
                            const float m = r == 0 ? mk[kk] : (r == 1 ? mk[3 + kk] : mk[6 + kk]);
                            const float sy = (float)(mpy + r - 1) + dy, sx = (float)(mpx + kk - 1) + dx;
                            if (sy > -1.f && sy < (float)H && sx > -1.f && sx < (float)W) {
                                const float fy = floorf(sy), fx = floorf(sx);
                                const int y0 = (int)fy, x0 = (int)fx;
                                const float ly = sy - fy, lx = sx - fx, hy = 1.f - ly, hx = 1.f - lx;
                                const bool yl = y0 >= 0, yh = y0 + 1 < H, xl = x0 >= 0, xh = x0 + 1 < W;
                                const int o00 = (y0 * W + x0) * Cin, o10 = o00 + W * Cin;
                                // rows y0 and y0+1 are staged as a whole or not at all
                                const bool in0 = o00 - x0 * Cin >= e_lo && o00 - x0 * Cin < e_hi, in1 = o10 - x0 * Cin >= e_lo && o10 - x0 * Cin < e_hi;
                                if (yl && xl) aq.x = in0 ? static_cast<uint32_t>(sel0 + 2 * o00) : (OUTSIDE | static_cast<uint32_t>(o00));
                                if (yl && xh) aq.y = in0 ? static_cast<uint32_t>(sel0 + 2 * (o00 + Cin)) : (OUTSIDE | static_cast<uint32_t>(o00 + Cin));
                                if (yh && xl) aq.z = in1 ? static_cast<uint32_t>(sel0 + 2 * o10) : (OUTSIDE | static_cast<uint32_t>(o10));
                                if (yh && xh) aq.w = in1 ? static_cast<uint32_t>(sel0 + 2 * (o10 + Cin)) : (OUTSIDE | static_cast<uint32_t>(o10 + Cin));
                                out = (yl && !in0) || (yh && !in1);
                                const float w00 = hy * hx * m, w01 = hy * lx * m, w10 = ly * hx * m, w11 = ly * lx * m;
                                wq = make_uint4(pack2<T>(w00, w00), pack2<T>(w01, w01), pack2<T>(w10, w10), pack2<T>(w11, w11));
                            }
                        }
                        my_w[kk * 32 + lane] = wq;
                        my_a[kk * 32 + lane] = aq;
                        if (__any_sync(0xffffffffu, out)) slow |= 1u << kk;
                    }
                    __syncwarp();
                    if (slow == 0) {
                        // the common case, unrolled over the three taps so that the loads of one tap overlap the MMAs of the previous
#pragma unroll
                        for (int kk = 0; kk < 3; ++kk)
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt)
                                deform_tap<T, NT, ALIGN, false, KCT>(acc[mt], smem_mma, gimg, my_w + kk * 32, my_a + kk * 32, mt * 16 + g, Bs, 3 * r + kk, KC, Cin, lane);
                    } else {
#pragma unroll 1
                        for (int kk = 0; kk < 3; ++kk) {
                            const int k = 3 * r + kk;
                            if ((slow >> kk) & 1u) {
#pragma unroll
                                for (int mt = 0; mt < 2; ++mt)
                                    deform_tap<T, NT, ALIGN, true, KCT>(acc[mt], smem_mma, gimg, my_w + kk * 32, my_a + kk * 32, mt * 16 + g, Bs, k, KC, Cin, lane);
                            } else {
#pragma unroll
                                for (int mt = 0; mt < 2; ++mt)
                                    deform_tap<T, NT, ALIGN, false, KCT>(acc[mt], smem_mma, gimg, my_w + kk * 32, my_a + kk * 32, mt * 16 + g, Bs, k, KC, Cin, lane);
                            }
                        }
                    }
                }
            }

            // ---- epilogue: affine, activation, post scale; the warp's 32 pixels leave as one contiguous run --------
            const int es = p.y_f32 ? 4 : 2;
            const int npx = min(32, HW - wbase);
            const bool tiled = 32 * Cout * es + 16 <= SCRATCH_PER_WARP;
            unsigned char* ydst = reinterpret_cast<unsigned char*>(p.y) + ((size_t)b * HW + wbase) * Cout * es;
            // the tile sits in shared memory at the same offset from a 16-byte boundary as its destination
            const int mis = static_cast<int>(reinterpret_cast<uintptr_t>(ydst) & 15);
            unsigned char* tile = tiled ? my_tile + mis : ydst;
            const bool pair_ok = !(Cout & 1) && !(mis & 3);
            __syncwarp();                                      // the table is no longer read
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = (j >> 1) * 16 + g + 8 * (j & 1);
                if (row >= npx) continue;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int co = nt * 8 + 2 * t;
                    if (co >= Cout) continue;
                    float v0 = fmaf(acc[j >> 1][nt][2 * (j & 1)], ep[co], ep[COP + co]);
                    float v1 = fmaf(acc[j >> 1][nt][2 * (j & 1) + 1], ep[co + 1], ep[COP + co + 1]);
                    if (p.act == KAD_ACT_SILU) { v0 = v0 * sigmoidf_(v0); v1 = v1 * sigmoidf_(v1); }
                    v0 = fmaxf(v0, relu_floor) * ep[2 * COP + co];
                    v1 = fmaxf(v1, relu_floor) * ep[2 * COP + co + 1];
                    const bool two = co + 1 < Cout;
                    const size_t idx = (size_t)row * Cout + co;
                    if (p.y_f32) {
                        float* yo = reinterpret_cast<float*>(tile) + idx;
                        yo[0] = v0; if (two) yo[1] = v1;
                    } else {
                        T* yo = reinterpret_cast<T*>(tile) + idx;
                        if (pair_ok) *reinterpret_cast<uint32_t*>(yo) = pack2<T>(v0, v1);
                        else { yo[0] = from_f<T>(v0); if (two) yo[1] = from_f<T>(v1); }
                        v0 = to_f<T>(from_f<T>(v0)); v1 = to_f<T>(from_f<T>(v1));     // sums of what the next kernel reads back
                    }
                    psum[nt][0] += v0;
                    if (two) psum[nt][1] += v1;
                }
            }
            if (tiled) {
                __syncwarp();
                const int nb = npx * Cout * es;
                const int head = min(nb, (16 - mis) & 15), body = (nb - head) >> 4, tail = nb - head - (body << 4);
                const uint4* src = reinterpret_cast<const uint4*>(tile + head);
                uint4* dst = reinterpret_cast<uint4*>(ydst + head);
                for (int i = lane; i < body; i += 32) dst[i] = src[i];
                if (lane < (head >> 1)) reinterpret_cast<uint16_t*>(ydst)[lane] = reinterpret_cast<const uint16_t*>(tile)[lane];
                else if (lane >= 16 && lane - 16 < (tail >> 1))
                    reinterpret_cast<uint16_t*>(ydst + head + (body << 4))[lane - 16] = reinterpret_cast<const uint16_t*>(tile + head + (body << 4))[lane - 16];
            }
        }

        // ---- channel sums of the group (squeeze-excite mean), deterministic -------------------------------------------
        if (p.gap_partial) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    float v = psum[nt][i];
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    if (g == 0) red[warp * COP + nt * 8 + 2 * t + i] = v;
                }
            __syncthreads();
            if (tid < Cout) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < MMA_WARPS; ++w) s += red[w * COP + tid];
                p.gap_partial[((size_t)b * gpi + grp) * Cout + tid] = s;
            }
        }
    }
}

inline int pick_nt(int Cout) {
    const int n = (Cout + 7) / 8;
    return n <= 2 ? 2 : n <= 3 ? 3 : n <= 4 ? 4 : n <= 6 ? 6 : 8;
}

// Shared memory of one block without the staged rows.
inline size_t fixed_smem(int KC, int nt, int mode) {
    size_t s = (size_t)9 * KC * nt * 32 * 8 + (size_t)MMA_WARPS * SCRATCH_PER_WARP + (size_t)3 * nt * 8 * 4 + (size_t)MMA_WARPS * nt * 8 * 4 + ZERO_BYTES;
    if (mode >= 2) s += (size_t)9 * KC * NT_OFF * 32 * 8 + (size_t)MMA_WARPS * 32 * OFF_PITCH * 4 + 32 * 4;
    return s;
}
// Image rows a group of 256 consecutive pixels can span, + 10 for the reach of the LCSA's 11x1 window.
inline int lcsa_rm_rows(int H, int W) {
    int rows = (W + MMA_THREADS - 2) / W + 1;
    if (rows > H) rows = H;
    return rows + 10;
}
// Extra shared memory of the inline-mask mode: 11x1 taps and 1x1 weights ([Cp][12] each), the staged row means and, when
// `cols`, the column terms A (current image) and Sm ([W][Cp] each).
inline size_t lcsa_smem(int Cin, int H, int W, bool cols) {
    const int Cp = (Cin + 3) & ~3;
    return (size_t)2 * Cp * 48 + (size_t)lcsa_rm_rows(H, W) * Cp * 4 + (cols ? (size_t)2 * W * Cp * 4 : 0);
}
// The column terms are staged when that costs at most 24 KB (narrow maps, few channels: the detector's shapes).
inline bool lcsa_stage_cols(int Cin, int W) { return (size_t)2 * W * ((Cin + 3) & ~3) * 4 <= 24 * 1024; }
// Bytes for the staged rows with `margin` rows for the learned offsets (incl. alignment slack on both sides).
inline size_t window_smem(int H, int W, int Cin, int margin) {
    int rows = (W + MMA_THREADS - 2) / W + 1 + 2 + 2 * margin;      // rows 256 consecutive pixels span + halo + margin
    if (rows > H) rows = H;
    return (size_t)rows * W * Cin * 2 + 16 + 16 + 32;
}
constexpr size_t SMEM_ONE_BLOCK = 224 * 1024, SMEM_TWO_BLOCKS = 112 * 1024;

template <typename T, int NT, int MODE, int KCT>
int launch_mma_align(const MmaParams& p, dim3 grid, size_t smem, cudaStream_t st) {
#define KAD_MMA_LAUNCH(A)                                                                                             \
    {                                                                                                                 \
        auto kern = dsc_mma_kernel<T, NT, MODE, A, KCT>;                                                              \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_mma smem attribute: %s", cudaGetErrorString(e));         \
        kern<<<grid, MMA_THREADS, smem, st>>>(p);                                                                     \
    }
    if (p.align == 8) KAD_MMA_LAUNCH(8) else if (p.align == 4) KAD_MMA_LAUNCH(4) else KAD_MMA_LAUNCH(2)
#undef KAD_MMA_LAUNCH
    return KAD_OK;
}

template <typename T, int NT>
int launch_mma_mode(const MmaParams& p, int mode, dim3 grid, size_t smem, cudaStream_t st) {
    if (mode == 0) return launch_mma_align<T, NT, 0, 0>(p, grid, smem, st);
    if (mode == 1) return launch_mma_align<T, NT, 1, 0>(p, grid, smem, st);
    if (mode == 3) {
        if (NT == 2 && p.KC == 1) return launch_mma_align<T, NT, 3, (NT == 2 ? 1 : 0)>(p, grid, smem, st);
        if (NT == 3 && p.KC == 2) return launch_mma_align<T, NT, 3, (NT == 3 ? 2 : 0)>(p, grid, smem, st);
        return launch_mma_align<T, NT, 3, 0>(p, grid, smem, st);
    }
    // the fused kernel at the detector's widths (<= 16 channels: NT 2, one chunk; 17-24 channels: NT 3, two chunks) is
    // compiled with the chunk count as a constant: index arithmetic folds and the chunk loops unroll
    if (NT == 2 && p.KC == 1) return launch_mma_align<T, NT, 2, (NT == 2 ? 1 : 0)>(p, grid, smem, st);
    if (NT == 3 && p.KC == 2) return launch_mma_align<T, NT, 2, (NT == 3 ? 2 : 0)>(p, grid, smem, st);
    return launch_mma_align<T, NT, 2, 0>(p, grid, smem, st);
}

template <typename T>
int launch_mma_nt(const MmaParams& p, int nt, int mode, dim3 grid, size_t smem, cudaStream_t st) {
    switch (nt) {
        case 2: return launch_mma_mode<T, 2>(p, mode, grid, smem, st);
        case 3: return launch_mma_mode<T, 3>(p, mode, grid, smem, st);
        case 4: return launch_mma_mode<T, 4>(p, mode, grid, smem, st);
        case 6: return launch_mma_mode<T, 6>(p, mode, grid, smem, st);
        default: return launch_mma_mode<T, 8>(p, mode, grid, smem, st);
    }
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace

// channel sums are written per group of 256 pixels
int dsc_mma_tiles(int H, int W) { return (H * W + MMA_THREADS - 1) / MMA_THREADS; }

// The fused mode (the largest footprint) must fit with at least the 3x3 halo staged.
bool dsc_mma_supported(int Cin, int Cout, int dtype, int H, int W) {
    if (!((dtype == KAD_F16 || dtype == KAD_BF16) && Cin >= 4 && Cin <= 64 && Cout >= 1 && Cout <= 64 && H >= 1 && W >= 1)) return false;
    if ((long long)H * W * Cin >= (1ll << 30)) return false;
    const int nt = pick_nt(Cout);
    return fixed_smem((Cin + 15) / 16, nt, 2) + window_smem(H, W, Cin, 0) <= SMEM_ONE_BLOCK;
}

// Inline-mask mode: the fused mode's footprint plus the LCSA operands must fit with at least the 3x3 halo staged.
bool dsc_mma_inline_mask_supported(int Cin, int Cout, int dtype, int H, int W) {
    if (!dsc_mma_supported(Cin, Cout, dtype, H, W)) return false;
    return fixed_smem((Cin + 15) / 16, pick_nt(Cout), 3) + lcsa_smem(Cin, H, W, lcsa_stage_cols(Cin, W)) + window_smem(H, W, Cin, 0) <= SMEM_ONE_BLOCK;
}

int launch_dsc_mma(const KadDscArgs& a, cudaStream_t st) {
    const bool fused = a.offset_weight != nullptr;
    const bool inline_mask = a.lcsa_rowmean != nullptr;
    KAD_CHECK_ARG(!inline_mask || fused, "kad_dsc_forward: the in-kernel LCSA mask needs the fused offset convolution (offset_weight)");
    KAD_CHECK_ARG(!inline_mask || (a.lcsa_A && a.lcsa_Sm && a.lcsa_w2 && a.lcsa_b2 && a.lcsa_w3 && a.lcsa_b3), "kad_dsc_forward: LCSA operand missing");
    KAD_CHECK_ARG(!inline_mask || ((uintptr_t)a.lcsa_A % 16 == 0 && (uintptr_t)a.lcsa_Sm % 16 == 0), "kad_dsc_forward: lcsa_A / lcsa_Sm must be 16-byte aligned");
    if (inline_mask && !dsc_mma_inline_mask_supported(a.Cin, a.Cout, a.dtype, a.H, a.W))
        return fail(KAD_ERR_UNSUPPORTED, "kad_dsc_forward: the in-kernel LCSA mask does not fit shared memory for Cin=%d H=%d W=%d", a.Cin, a.H, a.W);
    const int mode = inline_mask ? 3 : (fused ? 2 : (a.offset ? 1 : 0));
    KAD_CHECK_ARG(mode != 0 || a.mask == nullptr, "kad_dsc_forward: the warp-MMA path takes a mask only together with offsets");
    KAD_CHECK_ARG((uintptr_t)a.x % 16 == 0, "kad_dsc_forward: the warp-MMA path needs x aligned to 16 bytes");
    KAD_CHECK_ARG((uintptr_t)a.y % 4 == 0, "kad_dsc_forward: the warp-MMA path needs y aligned to 4 bytes");
    MmaParams p{};
    p.x = a.x; p.offset = fused ? nullptr : a.offset; p.mask = a.mask; p.Wt = (const float*)a.weight;
    p.Woff = a.offset_weight; p.boff = a.offset_bias;
    if (inline_mask) p.mask = nullptr;
    p.scale = a.scale; p.shift = a.shift; p.post = a.post; p.y = a.y; p.gap_partial = a.gap_partial;
    p.H = a.H; p.W = a.W; p.Cin = a.Cin; p.Cout = a.Cout; p.KC = (a.Cin + 15) / 16; p.B = a.B;
    p.align = a.Cin % 4 == 0 ? 8 : (a.Cin % 2 == 0 ? 4 : 2);
    p.offset_f32 = a.offset_f32; p.mask_f32 = a.mask_f32; p.y_f32 = a.y_f32; p.act = a.act;
    p.l_rowmean = a.lcsa_rowmean; p.l_A = a.lcsa_A; p.l_Sm = a.lcsa_Sm; p.l_w2 = a.lcsa_w2; p.l_b2 = a.lcsa_b2; p.l_w3 = a.lcsa_w3; p.l_b3 = a.lcsa_b3;
    p.Cp = (a.Cin + 3) & ~3; p.rm_rows = lcsa_rm_rows(a.H, a.W); p.stage_cols = (inline_mask && lcsa_stage_cols(a.Cin, a.W)) ? 1 : 0;
    const int nt = pick_nt(a.Cout);
    size_t smem = fixed_smem(p.KC, nt, mode) + (inline_mask ? lcsa_smem(a.Cin, a.H, a.W, p.stage_cols != 0) : 0);
    // rows of margin for the learned offsets: as many as fit, at most 2 (none for the plain convolution); the narrow
    // variants (128 registers) keep two blocks per SM when the halo alone allows it
    const size_t soft = (nt <= 4 && smem + window_smem(a.H, a.W, a.Cin, 0) <= SMEM_TWO_BLOCKS) ? SMEM_TWO_BLOCKS : SMEM_ONE_BLOCK;
    p.win_margin = 0;
    for (int m = (mode == 0 ? 0 : 2); m > 0; --m)
        if (smem + window_smem(a.H, a.W, a.Cin, m) <= soft) { p.win_margin = m; break; }
    smem += window_smem(a.H, a.W, a.Cin, p.win_margin);
    const long long groups = (long long)dsc_mma_tiles(a.H, a.W) * a.B;
    const long long resident = (long long)sm_count() * (soft == SMEM_TWO_BLOCKS ? 2 : 1);
    dim3 grid((unsigned)(groups < resident ? groups : resident), 1, 1);
    const int rc = a.dtype == KAD_F16 ? launch_mma_nt<__half>(p, nt, mode, grid, smem, st) : launch_mma_nt<__nv_bfloat16>(p, nt, mode, grid, smem, st);
    if (rc) return rc;
    KAD_CHECK_LAUNCH("dsc_mma_kernel");
    return KAD_OK;
}

}  // namespace kad
