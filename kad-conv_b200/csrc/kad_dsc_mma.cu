// Deformable 3x3 convolution for SMALL channel counts (the detector's DSCs have 10-44 channels) on the warp-level
// tensor-core instruction (mma.sync m16n8k16, fp16/bf16 operands, fp32 accumulators), NHWC.
//
// Why not the tcgen05 implicit GEMM: with K = 9 taps x 10..44 channels and N <= 64 the contraction is tiny; what costs
// is the bilinear gather and its geometry, i.e. instruction issue. So the kernel keeps the instruction count per pixel low:
// lane l of a warp OWNS pixel l of the warp's 32 pixels. It computes the pixel's sampling geometry in registers (no table),
// gathers the four corners of a tap for all channels with 8-byte shared-memory loads, interpolates them with packed
// half-precision FMAs (fp32 for bf16) and stores the interpolated samples as one row of a per-warp A tile
// [32 pixels][taps of the chunk x channels] in shared memory; after a chunk of taps (one kernel row) the warp reads the
// tile back as MMA fragments with ldmatrix and contracts it against the weight fragments. A gather instruction therefore
// serves 32 pixels (the earlier form of this kernel, where the four lanes of an accumulator row gathered straight into the
// fragments, served 8) and the bilinear blend costs one operation per two channels and corner.
//
// Blocks are persistent (two per SM for the narrow variants) and walk over (image, group of 256 consecutive pixels);
// a warp owns 32 pixels of the group (two 16-row MMA tiles). The image rows a group can reach (its own rows, one row of
// 3x3 halo, a margin for the learned offsets) are one CONTIGUOUS range of the NHWC tensor; it is copied to shared
// memory with 16-byte cp.async, so HBM sees one coalesced pass over x and the gathers are shared-memory loads with
// 32-bit addresses. A corner outside the image points at a block of zeros; a corner outside the staged rows (a large
// learned offset) is read from global memory by that lane. Results leave through shared memory as well, so that a warp
// writes its 32 pixels as one contiguous run.
//
// K layout of a tap: channels in groups of four (one 8-byte load); when Cin is no multiple of four the last group re-reads the
// last four channels of the pixel and the weight fragments carry zeros for the slots that would count a channel twice.
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
    int H, W, Cin, Cout, align;
    int G, KT, TPC, KS, pitchA, scratch;   // channel groups per tap, K slots per tap (4G), taps per chunk, 16-wide k-steps per chunk,
                                          // bytes per A-tile row, bytes of per-warp scratch (A tile, later the output tile)
    int offset_f32, mask_f32, y_f32, act;
    int B, win_margin;                  // win_margin: rows staged above / below the 3x3 halo for the learned offsets
    // inline mode: LCSA operands. rowmean [B][H][Cin] (means over x), A [B][W][Cp], Sm [W][Cp] (Cp = Cin rounded up to 4),
    // w2 [Cin][11], b2 [Cin], w3 [9][Cin], b3 [9]
    const float* l_rowmean; const float* l_A; const float* l_Sm; const float* l_w2; const float* l_b2; const float* l_w3; const float* l_b3;
    int Cp, rm_rows;                    // rm_rows: image rows a group of 256 pixels can span, + 10 for the 11x1 window
    int stage_cols;                     // 1: the image's A rows and Sm are staged in shared memory (they fit); 0: read through L2
    const uint4* frags; int frag_vecs;  // fused mode, optional: the weight fragments of both convolutions as kad_dsc_mma_pack_frags wrote them, in 16-byte units
};

constexpr int ZERO_BYTES = 160;         // block of zeros in shared memory that out-of-image corners point at

// First channel of channel group j of a pixel (see the K layout above).
__device__ __forceinline__ int group_first(int j, int Cin) {
    const int ch = 4 * j, nv = Cin - ch;
    return nv >= 4 ? ch : Cin - 4;
}

// Weight fragments for mma.sync, per chunk of TPC taps: dst [9 / TPC][KS][NT][32 lanes]. Lane (g = lane / 4, t = lane % 4) of
// n-tile nt holds output channel nt*8 + g and the K slots ks*16 + {2t, 2t+1, 2t+8, 2t+9} of the chunk; slot = tap_in_chunk * KT +
// 4*group + i stands for channel group_first(group) + i of that tap, and is zero when the slot is padding or repeats a channel.
template <typename T>
__device__ __forceinline__ void stage_weights(uint2* dst, const float* __restrict__ Wt, int Cin, int Cout, int KT, int TPC, int KS, int NT, int tid) {
    const int total = (9 / TPC) * KS * NT * 32;
    for (int e = tid; e < total; e += MMA_THREADS) {
        const int lane = e & 31, f = e >> 5, nt = f % NT, ks = (f / NT) % KS, ch = f / (NT * KS);
        const int n = nt * 8 + (lane >> 2), t = lane & 3;
        const int kk[4] = {ks * 16 + 2 * t, ks * 16 + 2 * t + 1, ks * 16 + 2 * t + 8, ks * 16 + 2 * t + 9};
        float w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int tl = kk[i] / KT, slot = kk[i] - tl * KT, j = slot >> 2, c = group_first(j, Cin) + (slot & 3);
            const bool ok = tl < TPC && n < Cout && c >= 4 * j;
            w[i] = ok ? Wt[((size_t)(ch * TPC + tl) * Cin + c) * Cout + n] : 0.f;
        }
        dst[e] = make_uint2(pack2<T>(w[0], w[1]), pack2<T>(w[2], w[3]));
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// acc += A tile (32 rows x KS*16, rows pitchA bytes apart, at shared-memory address `tile`) x the chunk's weight fragments.
template <typename T, int NTP>
__device__ __forceinline__ void mma_chunk(float (&acc)[2][NTP][4], uint32_t tile, int pitchA, const uint2* __restrict__ Bc, int KS, int lane) {
    // ldmatrix x4 of a 16 x 16 block: lanes 0-15 address rows 0-15 at k 0-7, lanes 16-31 the same rows at k 8-15
    const uint32_t a0 = tile + (uint32_t)((lane & 15) * pitchA + (lane >> 4) * 16);
#pragma unroll 1
    for (int ks = 0; ks < KS; ++ks) {
        uint2 bf[NTP];
#pragma unroll
        for (int nt = 0; nt < NTP; ++nt) bf[nt] = Bc[(ks * NTP + nt) * 32 + lane];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(a0 + (uint32_t)(mt * 16 * pitchA + ks * 32), r0, r1, r2, r3);
#pragma unroll
            for (int nt = 0; nt < NTP; ++nt) mma16816<T>(acc[mt][nt], r0, r1, r2, r3, bf[nt]);
        }
    }
}

// Bilinear blend of four corners, four channels at a time; weights are the mask-scaled corner weights.
template <typename T> struct CornerWeights;
template <> struct CornerWeights<__half> {
    uint32_t w[4];
    __device__ __forceinline__ void set(float a, float b, float c, float d) {
        w[0] = pack2<__half>(a, a); w[1] = pack2<__half>(b, b); w[2] = pack2<__half>(c, c); w[3] = pack2<__half>(d, d);
    }
    __device__ __forceinline__ uint32_t blend(uint32_t a, uint32_t b, uint32_t c, uint32_t d) const {
        const __half2* pw = reinterpret_cast<const __half2*>(w);
        __half2 r = __hmul2(pw[0], *reinterpret_cast<__half2*>(&a));
        r = __hfma2(pw[1], *reinterpret_cast<__half2*>(&b), r);
        r = __hfma2(pw[2], *reinterpret_cast<__half2*>(&c), r);
        r = __hfma2(pw[3], *reinterpret_cast<__half2*>(&d), r);
        return *reinterpret_cast<uint32_t*>(&r);
    }
};
template <> struct CornerWeights<__nv_bfloat16> {      // bf16 has 8 bits of mantissa: blend in float32, round once
    float w[4];
    __device__ __forceinline__ void set(float a, float b, float c, float d) { w[0] = a; w[1] = b; w[2] = c; w[3] = d; }
    __device__ __forceinline__ uint32_t blend(uint32_t a, uint32_t b, uint32_t c, uint32_t d) const {
        const float2 fa = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&a)), fb = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&b));
        const float2 fc = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&c)), fd = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&d));
        return pack2<__nv_bfloat16>(fmaf(w[3], fd.x, fmaf(w[2], fc.x, fmaf(w[1], fb.x, w[0] * fa.x))),
                                    fmaf(w[3], fd.y, fmaf(w[2], fc.y, fmaf(w[1], fb.y, w[0] * fa.y))));
    }
};

// One tap of one pixel: gather the four corners group by group, blend, store at `dst` (the tap's slots of the pixel's A-tile row).
// aq: shared-memory byte offsets of the four corners (always inside the staged rows). SLOW (some lane of the warp has a corner in
// an image row that is not staged): such a corner, marked in `far` (bit cr), is read from global memory at element offset ge[cr].
template <typename T, int ALIGN, bool SLOW, int GT>
__device__ __forceinline__ void gather_tap(unsigned char* dst, const unsigned char* smem, const unsigned char* gimg, const uint32_t (&aq)[4],
                                           uint32_t far, const int (&ge)[4], const CornerWeights<T>& cw, int Gr, int Cin) {
    const int G = GT ? GT : Gr;
    if (ALIGN == 16) {
        // Cin is a multiple of 8 and every pixel starts on a 16-byte boundary: eight channels per load. (With 32-byte pixel strides
        // 8-byte loads of 32 neighbouring pixels hit only four bank positions; 16-byte loads halve both the conflicts and the loads.)
#pragma unroll (GT ? GT / 2 : 1)
        for (int j = 0; j < (G >> 1); ++j) {
            uint4 v[4];
#pragma unroll
            for (int cr = 0; cr < 4; ++cr) {
                if (SLOW && ((far >> cr) & 1u)) v[cr] = __ldg(reinterpret_cast<const uint4*>(gimg + 2 * (size_t)ge[cr] + 16 * j));
                else v[cr] = *reinterpret_cast<const uint4*>(smem + aq[cr] + 16u * (uint32_t)j);
            }
            *reinterpret_cast<uint4*>(dst + 16 * j) = make_uint4(cw.blend(v[0].x, v[1].x, v[2].x, v[3].x), cw.blend(v[0].y, v[1].y, v[2].y, v[3].y),
                                                                  cw.blend(v[0].z, v[1].z, v[2].z, v[3].z), cw.blend(v[0].w, v[1].w, v[2].w, v[3].w));
        }
        return;
    }
#pragma unroll (GT ? GT : 1)
    for (int j = 0; j < G; ++j) {
        // with GT known, Cin lies in (4*(GT-1), 4*GT]: every group but the last starts at channel 4*j (a constant offset)
        const uint32_t coff = (GT && j < GT - 1) ? 8u * (uint32_t)j : 2u * (uint32_t)group_first(j, Cin);
        uint2 v[4];
#pragma unroll
        for (int cr = 0; cr < 4; ++cr) {
            if (SLOW && ((far >> cr) & 1u)) v[cr] = ldg8<ALIGN>(gimg + 2 * (size_t)ge[cr] + coff);
            else v[cr] = lds8<ALIGN>(smem, aq[cr] + coff);
        }
        *reinterpret_cast<uint2*>(dst + 8 * j) = make_uint2(cw.blend(v[0].x, v[1].x, v[2].x, v[3].x), cw.blend(v[0].y, v[1].y, v[2].y, v[3].y));
    }
}

// Ordinary zero-padded 3x3 convolution (the offset convolution; the whole kernel in plain mode). No A tile here: without
// deformation the four lanes that share an accumulator row load four channels each straight into the A fragment registers, and
// a 3x3 convolution has no geometry to compute, so that form has the fewest instructions. Its weight fragments use a K order
// permuted to match: lane t of a 16-channel chunk holds four CONSECUTIVE channels (logical k = 2t, 2t+1, 2t+8, 2t+9 <-> channel
// lane_first_channel() + 0..3), layout [9 taps][KC chunks][NT][32 lanes].
template <typename T>
__device__ __forceinline__ void stage_weights_rows(uint2* dst, const float* __restrict__ Wt, int Cin, int Cout, int KC, int NT, int tid) {
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

// so[j] = shared-memory address of the pixel of this lane's accumulator row j, vm[j] = which of its 9 neighbours lie inside the image.
// KCT: the number of 16-channel chunks when it is known at compile time, 0 = use KCr.
template <typename T, int NTP, int ALIGN, int KCT>
__device__ __forceinline__ void plain_pass(float (&acc)[2][NTP][4], const unsigned char* smem, const uint32_t (&so)[4], const uint32_t (&vm)[4],
                                           uint32_t zoff, const uint2* __restrict__ Bw, int KCr, int Cin, int W, int lane) {
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
            for (int nt = 0; nt < NTP; ++nt) bf[nt] = Bw[((k * KC + kc) * NTP + nt) * 32 + lane];
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
    for (int j = 0; j < 9; ++j) mk[j] = sigmoid_mask(logit[j]);
}

template <typename T, int NT, int MODE, int ALIGN, int GT>       // MODE 0 plain, 1 deform, 2 fused, 3 fused + inline LCSA mask; GT: channel groups per tap when known at compile time
__global__ void __launch_bounds__(MMA_THREADS, NT <= 4 ? 2 : 1)
dsc_mma_kernel(const MmaParams p) {
    constexpr int COP = NT * 8;
    extern __shared__ __align__(16) unsigned char smem_mma[];
    constexpr bool FUSED = MODE >= 2, INLINE = MODE == 3;
    constexpr int KCT = GT ? (GT + 3) / 4 : 0;                                        // 16-channel chunks of the plain passes, if known
    const int nch = 9 / p.TPC, KS = p.KS, KC = KCT ? KCT : (p.Cin + 15) / 16;
    uint2* Bs = reinterpret_cast<uint2*>(smem_mma);                                   // deform: [nch][KS][NT][32]; plain mode: [9][KC][NT][32]
    uint2* Bo = Bs + (MODE == 0 ? 9 * KC : nch * KS) * NT * 32;                       // [9][KC][3][32]   (fused: the offset convolution)
    unsigned char* cur = reinterpret_cast<unsigned char*>(Bo + (FUSED ? 9 * KC * NT_OFF * 32 : 0));
    unsigned char* scratch = cur; cur += MMA_WARPS * p.scratch;
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

    unsigned char* my_tile = scratch + warp * p.scratch;                              // the warp's A tile; after the taps its output tile
    unsigned char* my_row = my_tile + lane * p.pitchA;                                // this lane's pixel's row of the A tile
    const uint32_t my_tile_addr = static_cast<uint32_t>(__cvta_generic_to_shared(my_tile));
    float* my_offs = offs + warp * 32 * OFF_PITCH;
    const float relu_floor = p.act == KAD_ACT_RELU ? 0.f : -INFINITY;

    // ---- parameters first: weight fragments, epilogue vectors, the block of zeros. Nothing here was written by another kernel, so
    // with a programmatic launch this part runs while the kernel before this one is still draining ----------------------------------
    if (MODE == 2 && p.frags) {
        // fragments packed once by kad_dsc_mma_pack_frags: a straight copy (both convolutions lie one after the other, as here);
        // the copy is waited for together with the first group's image rows
        uint4* dst = reinterpret_cast<uint4*>(Bs);
        for (int i = tid; i < p.frag_vecs; i += MMA_THREADS) cp_async16(dst + i, p.frags + i);
    } else {
        if (MODE == 0) stage_weights_rows<T>(Bs, p.Wt, Cin, Cout, KC, NT, tid);
        else stage_weights<T>(Bs, p.Wt, Cin, Cout, p.KT, p.TPC, KS, NT, tid);
        if (FUSED) stage_weights_rows<T>(Bo, p.Woff, Cin, 18, KC, NT_OFF, tid);
    }
    if (FUSED && tid < 24) boffs[tid] = (tid < 18 && p.boff) ? p.boff[tid] : 0.f;
    if (INLINE) {
        for (int e = tid; e < 12 * p.Cp; e += MMA_THREADS) {
            const int c = e / 12, k = e - c * 12;
            sw3[e] = (k < 9 && c < Cin) ? p.l_w3[k * Cin + c] : 0.f;
            sw2[e] = c < Cin ? (k < 11 ? p.l_w2[c * 11 + k] : p.l_b2[c]) : 0.f;
        }
    }
    for (int e = tid; e < COP; e += MMA_THREADS) {
        const bool on = e < Cout;
        ep[e] = (on && p.scale) ? p.scale[e] : 1.f;
        ep[COP + e] = (on && p.shift) ? p.shift[e] : 0.f;
        ep[2 * COP + e] = (on && p.post) ? p.post[e] : 1.f;
    }
    if (tid < ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(smem_mma + zoff)[tid] = 0u;
    grid_dependency_wait();              // x, offsets, mask and the LCSA vectors come from the kernels before
    grid_dependents_go();

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
            if (INLINE && p.stage_cols) for (int e = tid; e < W * p.Cp; e += MMA_THREADS) Sms[e] = p.l_Sm[e];
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
            float acc[2][NT][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

            if (MODE == 0 || FUSED) {
                // plain passes work on accumulator rows: j = mt*2 + half -> pixel wbase + mt*16 + g + 8*half
                uint32_t so4[4], vm4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int rr = (j >> 1) * 16 + g + 8 * (j & 1);
                    vm4[j] = __shfl_sync(0xffffffffu, myvm, rr);
                    so4[j] = static_cast<uint32_t>(sel0 + 2 * (wbase + rr) * Cin);
                }
                if (MODE == 0) {
                    plain_pass<T, NT, ALIGN, KCT>(acc, smem_mma, so4, vm4, zoff, Bs, KC, Cin, W, lane);
                } else {
                    // offset convolution of the warp's 32 pixels -> shared memory [32][18]
                    float oacc[2][NT_OFF][4];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int nt = 0; nt < NT_OFF; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) oacc[mt][nt][i] = 0.f;
                    plain_pass<T, NT_OFF, ALIGN, KCT>(oacc, smem_mma, so4, vm4, zoff, Bo, KC, Cin, W, lane);
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
            }
            if (MODE != 0) {
                // K slots of this lane's A-tile row beyond the chunk's taps are never written by the gather; their weights are zero, but
                // what the previous group's output tile left there may not be a finite number: clear them
                for (int o = p.TPC * p.KT * 2; o < KS * 32; o += 8) *reinterpret_cast<uint2*>(my_row + o) = make_uint2(0u, 0u);
                // Sampling geometry of this lane's pixel, per tap, in registers. A corner outside the image gets weight 0 and its
                // coordinates are clamped, so every address is valid; rows are clamped to the STAGED rows [ys0, ys1], and a corner
                // that lies in the image but in a row that is not staged (a large offset) is flagged and read from global memory.
                const int ys0 = e_lo / (W * Cin), ys1 = e_hi / (W * Cin) - 1;
                const uint32_t row_bytes = 2u * (uint32_t)(W * Cin), px_bytes = 2u * (uint32_t)Cin;
                const uint32_t s00 = static_cast<uint32_t>(sel0);
                const float fy0 = (float)(mpy - 1), fx0 = (float)(mpx - 1);
                auto tap = [&](int k, int tl) {
                    const int r = k / 3, kk = k - 3 * r;
                    float dy, dx;
                    if (FUSED) { dy = my_offs[lane * OFF_PITCH + 2 * k]; dx = my_offs[lane * OFF_PITCH + 2 * k + 1]; }
                    else { dy = load_mixed<T>(p.offset, gp * 18 + 2 * k, p.offset_f32); dx = load_mixed<T>(p.offset, gp * 18 + 2 * k + 1, p.offset_f32); }
                    float m = mk[0];
#pragma unroll
                    for (int q = 1; q < 9; ++q) m = (k == q) ? mk[q] : m;         // folds when the tap loops are unrolled
                    const float sy = (fy0 + (float)r) + dy, sx = (fx0 + (float)kk) + dx;
                    const float fy = floorf(sy), fx = floorf(sx);
                    const float ly = sy - fy, lx = sx - fx;
                    // saturating conversions: a sample far outside the image ends with all four corners invalid
                    const int y0 = __float2int_rd(fminf(fmaxf(sy, -4.f), (float)H + 2.f)), x0 = __float2int_rd(fminf(fmaxf(sx, -4.f), (float)W + 2.f));
                    const bool yl = (unsigned)y0 < (unsigned)H, yh = (unsigned)(y0 + 1) < (unsigned)H;
                    const bool xl = (unsigned)x0 < (unsigned)W, xh = (unsigned)(x0 + 1) < (unsigned)W;
                    const float wy0 = (yl && mylive) ? (1.f - ly) * m : 0.f, wy1 = (yh && mylive) ? ly * m : 0.f;
                    const float wx0 = xl ? 1.f - lx : 0.f, wx1 = xh ? lx : 0.f;
                    CornerWeights<T> cw;
                    cw.set(wy0 * wx0, wy0 * wx1, wy1 * wx0, wy1 * wx1);
                    const int r0 = min(max(y0, ys0), ys1), r1 = min(max(y0 + 1, ys0), ys1);
                    const int c0 = min(max(x0, 0), W - 1), c1 = min(max(x0 + 1, 0), W - 1);
                    const uint32_t a0 = s00 + (uint32_t)r0 * row_bytes, a1 = s00 + (uint32_t)r1 * row_bytes;
                    const uint32_t b0 = (uint32_t)c0 * px_bytes, b1 = (uint32_t)c1 * px_bytes;
                    const uint32_t aq[4] = {a0 + b0, a0 + b1, a1 + b0, a1 + b1};
                    // corners with weight in an image row outside the staged ones
                    const bool far0 = mylive && yl && r0 != y0, far1 = mylive && yh && r1 != y0 + 1;
                    unsigned char* dst = my_row + tl * p.KT * 2;
                    if (!__any_sync(0xffffffffu, far0 || far1)) {
                        const int ge[4] = {0, 0, 0, 0};
                        gather_tap<T, ALIGN, false, GT>(dst, smem_mma, gimg, aq, 0u, ge, cw, p.G, Cin);
                    } else {
                        const uint32_t far = (far0 ? 3u : 0u) | (far1 ? 12u : 0u);
                        const int g0 = (min(max(y0, 0), H - 1) * W) * Cin, g1 = (min(max(y0 + 1, 0), H - 1) * W) * Cin;
                        const int ge[4] = {g0 + c0 * Cin, g0 + c1 * Cin, g1 + c0 * Cin, g1 + c1 * Cin};
                        gather_tap<T, ALIGN, true, GT>(dst, smem_mma, gimg, aq, far, ge, cw, p.G, Cin);
                    }
                };
                if (GT) {          // three taps per chunk (GT <= 6 groups), everything unrolled
#pragma unroll
                    for (int ch = 0; ch < 3; ++ch) {
                        __syncwarp();                          // the previous chunk's fragments have been read; the offsets are visible
#pragma unroll
                        for (int tl = 0; tl < 3; ++tl) tap(3 * ch + tl, tl);
                        __syncwarp();
                        mma_chunk<T, NT>(acc, my_tile_addr, p.pitchA, Bs + (size_t)ch * KS * NT * 32, KS, lane);
                    }
                } else {
#pragma unroll 1
                    for (int ch = 0; ch < nch; ++ch) {
                        __syncwarp();
#pragma unroll 1
                        for (int tl = 0; tl < p.TPC; ++tl) tap(ch * p.TPC + tl, tl);
                        __syncwarp();
                        mma_chunk<T, NT>(acc, my_tile_addr, p.pitchA, Bs + (size_t)ch * KS * NT * 32, KS, lane);
                    }
                }
            }

            // ---- epilogue: affine, activation, post scale; the warp's 32 pixels leave as one contiguous run --------
            const int es = p.y_f32 ? 4 : 2;
            const int npx = min(32, HW - wbase);
            const bool tiled = 32 * Cout * es + 16 <= p.scratch;
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

// The weight fragments of the fused mode (deformable convolution, then offset convolution) written to global memory once, in the
// order the kernel keeps them in shared memory, so that every block of every launch copies them instead of deriving them.
template <typename T>
__global__ void __launch_bounds__(MMA_THREADS)
pack_frags_kernel(uint2* __restrict__ dst, const float* __restrict__ Wt, const float* __restrict__ Woff, int Cin, int Cout, int KT, int TPC, int KS, int NT, int KC) {
    stage_weights<T>(dst, Wt, Cin, Cout, KT, TPC, KS, NT, threadIdx.x);
    stage_weights_rows<T>(dst + (9 / TPC) * KS * NT * 32, Woff, Cin, 18, KC, NT_OFF, threadIdx.x);
}

// K structure of the A tile for Cin channels: groups of four channels per tap, taps per chunk (a kernel row of three taps while
// its K stays <= 80, i.e. up to 24 channels, else single taps), 16-wide k-steps per chunk, row pitch (an odd number of 16-byte units, so that the eight
// rows of an ldmatrix phase hit different banks) and the per-warp scratch (A tile or output tile, whichever is larger).
struct KPlan { int G, KT, TPC, KS, pitchA, scratch; };
inline KPlan k_plan(int Cin, int Cout) {
    KPlan k;
    k.G = (Cin + 3) / 4; k.KT = 4 * k.G;
    k.TPC = 3 * k.KT <= 80 ? 3 : 1;
    k.KS = (k.TPC * k.KT + 15) / 16;
    k.pitchA = k.KS * 32 + 16;
    const int tile = 32 * k.pitchA, outt = 32 * Cout * 4 + 16;
    k.scratch = ((tile > outt ? tile : outt) + 15) & ~15;
    return k;
}
// Shared memory of one block without the staged rows.
inline size_t fixed_smem(int Cin, int Cout, int nt, int mode) {
    const KPlan k = k_plan(Cin, Cout);
    const size_t frag = (size_t)(9 / k.TPC) * k.KS * 32 * 8;          // bytes of weight fragments per n-tile, deformable passes
    const size_t frag_rows = (size_t)9 * ((Cin + 15) / 16) * 32 * 8;  // the same for the plain passes
    size_t s = (mode == 0 ? frag_rows : frag) * nt + (size_t)MMA_WARPS * k.scratch + (size_t)3 * nt * 8 * 4 + (size_t)MMA_WARPS * nt * 8 * 4 + ZERO_BYTES;
    if (mode >= 2) s += frag_rows * NT_OFF + (size_t)MMA_WARPS * 32 * OFF_PITCH * 4 + 32 * 4;
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

template <typename T, int NT, int MODE, int GT>
int launch_mma_align(const MmaParams& p, dim3 grid, size_t smem, cudaStream_t st) {
#define KAD_MMA_LAUNCH(A)                                                                                             \
    {                                                                                                                 \
        auto kern = dsc_mma_kernel<T, NT, MODE, A, GT>;                                                              \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "dsc_mma smem attribute: %s", cudaGetErrorString(e));         \
        launch_pdl(kern, grid, MMA_THREADS, smem, st, p);                                                            \
    }
    if (p.align == 16) KAD_MMA_LAUNCH(16) else if (p.align == 8) KAD_MMA_LAUNCH(8) else if (p.align == 4) KAD_MMA_LAUNCH(4) else KAD_MMA_LAUNCH(2)
#undef KAD_MMA_LAUNCH
    return KAD_OK;
}

template <typename T, int NT>
int launch_mma_mode(const MmaParams& p, int mode, dim3 grid, size_t smem, cudaStream_t st) {
    if (mode == 0) return launch_mma_align<T, NT, 0, 0>(p, grid, smem, st);
    if (mode == 1) return launch_mma_align<T, NT, 1, 0>(p, grid, smem, st);
    // the fused kernels at the detector's widths (9-12 and 13-16 channels: NT 2, three / four channel groups; 21-24 channels: NT 3,
    // six groups) are compiled with the group count as a constant: the gather loops unroll and their addresses fold
    if (mode == 3) {
        if (NT == 2 && p.G == 3) return launch_mma_align<T, NT, 3, (NT == 2 ? 3 : 0)>(p, grid, smem, st);
        if (NT == 2 && p.G == 4) return launch_mma_align<T, NT, 3, (NT == 2 ? 4 : 0)>(p, grid, smem, st);
        if (NT == 3 && p.G == 6) return launch_mma_align<T, NT, 3, (NT == 3 ? 6 : 0)>(p, grid, smem, st);
        return launch_mma_align<T, NT, 3, 0>(p, grid, smem, st);
    }
    if (NT == 2 && p.G == 3) return launch_mma_align<T, NT, 2, (NT == 2 ? 3 : 0)>(p, grid, smem, st);
    if (NT == 2 && p.G == 4) return launch_mma_align<T, NT, 2, (NT == 2 ? 4 : 0)>(p, grid, smem, st);
    if (NT == 3 && p.G == 6) return launch_mma_align<T, NT, 2, (NT == 3 ? 6 : 0)>(p, grid, smem, st);
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

// bytes of the fragment image of the fused mode: (9 / TPC) * KS * NT deformable + 9 * KC * NT_OFF offset fragments of 32 lanes x 8 bytes
size_t dsc_mma_frag_bytes(int Cin, int Cout) {
    const KPlan k = k_plan(Cin, Cout);
    return ((size_t)(9 / k.TPC) * k.KS * pick_nt(Cout) + (size_t)9 * ((Cin + 15) / 16) * NT_OFF) * 32 * 8;
}

int dsc_mma_pack_frags(const float* w_simt, const float* w_off_simt, void* dst, int Cin, int Cout, int dtype, cudaStream_t st) {
    const KPlan k = k_plan(Cin, Cout);
    const int nt = pick_nt(Cout), KC = (Cin + 15) / 16;
    if (dtype == KAD_F16) pack_frags_kernel<__half><<<1, MMA_THREADS, 0, st>>>((uint2*)dst, w_simt, w_off_simt, Cin, Cout, k.KT, k.TPC, k.KS, nt, KC);
    else pack_frags_kernel<__nv_bfloat16><<<1, MMA_THREADS, 0, st>>>((uint2*)dst, w_simt, w_off_simt, Cin, Cout, k.KT, k.TPC, k.KS, nt, KC);
    KAD_CHECK_LAUNCH("pack_frags_kernel");
    return KAD_OK;
}

// channel sums are written per group of 256 pixels
int dsc_mma_tiles(int H, int W) { return (H * W + MMA_THREADS - 1) / MMA_THREADS; }

// The fused mode (the largest footprint) must fit with at least the 3x3 halo staged.
bool dsc_mma_supported(int Cin, int Cout, int dtype, int H, int W) {
    if (!((dtype == KAD_F16 || dtype == KAD_BF16) && Cin >= 4 && Cin <= 64 && Cout >= 1 && Cout <= 64 && H >= 1 && W >= 1)) return false;
    if ((long long)H * W * Cin >= (1ll << 30)) return false;
    const int nt = pick_nt(Cout);
    return fixed_smem(Cin, Cout, nt, 2) + window_smem(H, W, Cin, 0) <= SMEM_ONE_BLOCK;
}

// Inline-mask mode: the fused mode's footprint plus the LCSA operands must fit with at least the 3x3 halo staged.
bool dsc_mma_inline_mask_supported(int Cin, int Cout, int dtype, int H, int W) {
    if (!dsc_mma_supported(Cin, Cout, dtype, H, W)) return false;
    return fixed_smem(Cin, Cout, pick_nt(Cout), 3) + lcsa_smem(Cin, H, W, lcsa_stage_cols(Cin, W)) + window_smem(H, W, Cin, 0) <= SMEM_ONE_BLOCK;
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
    p.H = a.H; p.W = a.W; p.Cin = a.Cin; p.Cout = a.Cout; p.B = a.B;
    { const KPlan k = k_plan(a.Cin, a.Cout); p.G = k.G; p.KT = k.KT; p.TPC = k.TPC; p.KS = k.KS; p.pitchA = k.pitchA; p.scratch = k.scratch; }
    p.align = a.Cin % 8 == 0 ? 16 : (a.Cin % 4 == 0 ? 8 : (a.Cin % 2 == 0 ? 4 : 2));
    p.offset_f32 = a.offset_f32; p.mask_f32 = a.mask_f32; p.y_f32 = a.y_f32; p.act = a.act;
    p.l_rowmean = a.lcsa_rowmean; p.l_A = a.lcsa_A; p.l_Sm = a.lcsa_Sm; p.l_w2 = a.lcsa_w2; p.l_b2 = a.lcsa_b2; p.l_w3 = a.lcsa_w3; p.l_b3 = a.lcsa_b3;
    p.Cp = (a.Cin + 3) & ~3; p.rm_rows = lcsa_rm_rows(a.H, a.W); p.stage_cols = (inline_mask && lcsa_stage_cols(a.Cin, a.W)) ? 1 : 0;
    const int nt = pick_nt(a.Cout);
    if (mode == 2 && a.mma_frags) {
        KAD_CHECK_ARG((uintptr_t)a.mma_frags % 16 == 0, "kad_dsc_forward: mma_frags must be 16-byte aligned");
        p.frags = reinterpret_cast<const uint4*>(a.mma_frags);
        p.frag_vecs = (int)(dsc_mma_frag_bytes(a.Cin, a.Cout) / 16);
    }
    size_t smem = fixed_smem(a.Cin, a.Cout, nt, mode) + (inline_mask ? lcsa_smem(a.Cin, a.H, a.W, p.stage_cols != 0) : 0);
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
