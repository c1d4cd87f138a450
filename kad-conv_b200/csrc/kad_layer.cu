// One C-ABI call for a whole KAD-Conv layer (KADConv.forward of the reference, KAD-Conv/kadconv/kad_conv.py:112-121):
// the three branches are independent until the final concat, so they are issued on three streams (the caller's stream
// and two library-owned side streams, forked and joined with events) and run concurrently; under stream capture
// the fork/join becomes three parallel chains of one CUDA graph. All intermediate tensors live in a workspace the
// caller provides, so nothing is allocated per call.
#include <mutex>

#include "kad_common.cuh"

namespace kad {
namespace {

struct SideStreams {
    cudaStream_t s[2] = {nullptr, nullptr};
    cudaEvent_t fork = nullptr, join[2] = {nullptr, nullptr};
    bool ready = false;
};
constexpr int MAX_DEVICES = 64;
SideStreams g_side[MAX_DEVICES];
std::mutex g_side_mutex;

int side_streams(int dev, SideStreams** out) {
    std::lock_guard<std::mutex> lock(g_side_mutex);
    SideStreams& ss = g_side[dev];
    if (!ss.ready) {
        // the pooled branches run on streams of the LOWEST priority: the full-resolution branch on the caller's stream is the
        // longest chain of a layer, and its blocks should get an SM first when both have blocks waiting
        int prio_lo = 0, prio_hi = 0;
        cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);        // numerically lowest = highest priority
        for (int i = 0; i < 2; ++i) {
            cudaError_t e = cudaStreamCreateWithPriority(&ss.s[i], cudaStreamNonBlocking, prio_lo);
            if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: side stream: %s", cudaGetErrorString(e));
            e = cudaEventCreateWithFlags(&ss.join[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: event: %s", cudaGetErrorString(e));
        }
        cudaError_t e = cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: event: %s", cudaGetErrorString(e));
        ss.ready = true;
    }
    *out = &ss;
    return KAD_OK;
}

inline size_t align_up(size_t v) { return (v + 255) & ~size_t(255); }

struct BranchWs {
    size_t t, rows, cols, rowpart, colpart, scratch, mask, offset, y, gap, att, end;
};

BranchWs plan_branch(size_t base, int B, int h, int w, int c, size_t es, int gap_tiles, int nct, int nrg) {
    BranchWs p;
    size_t o = base;
    p.t = o; o = align_up(o + (size_t)B * h * w * c * es);
    p.rows = o; o = align_up(o + (size_t)B * h * c * 4);
    p.cols = o; o = align_up(o + (size_t)B * w * c * 4);
    p.rowpart = o; o = align_up(o + (size_t)B * h * nct * c * 4);     // partial sums of the pyramid kernel (nct = 0: unused)
    p.colpart = o; o = align_up(o + (size_t)B * nrg * w * c * 4);
    p.scratch = o; o = align_up(o + ((size_t)B + 1) * w * ((c + 3) & ~3) * 4);
    p.mask = o; o = align_up(o + (size_t)B * h * w * 9 * 4);
    p.offset = o; o = align_up(o + (size_t)B * h * w * 18 * 4);
    p.y = o; o = align_up(o + (size_t)B * h * w * c * es);
    p.gap = o; o = align_up(o + (size_t)B * gap_tiles * c * 4);
    p.att = o; o = align_up(o + (size_t)B * c * 4);
    p.end = o;
    return p;
}

// 1 = tcgen05 implicit GEMM, 3 = warp-MMA kernel with the offset convolution fused in, 0 = SIMT
int branch_path(const KadBranchParams& br, int dtype, int h, int w) {
    if (br.w_dsc_tc && kad_dsc_tc_supported(br.c, br.c, dtype)) return 1;
    return kad_dsc_mma_supported(br.c, br.c, dtype, h, w) ? 3 : 0;
}

// What the layer call does for this shape, and where everything lives in the workspace.
struct LayerPlan {
    BranchWs ws[3];
    int path[3], tiles[3];
    bool pyramid, partials;      // one kernel for the three projections; LCSA sums taken from that kernel's partial sums
    bool fused_lcsa;             // the three LCSAs can run as one launch from the partial sums
    bool tail_prep;              // LCSA first stage can be finished in the pyramid kernel's tail
    bool inline_mask;            // ... and the masks can be evaluated inside the deformable convolutions
    int nct, nrg;
    size_t bytes;
};

LayerPlan plan_layer(int B, int H, int W, int dim, int dtype, int tc_mask) {
    LayerPlan L{};
    const size_t es = dtype_size(dtype);
    const int widths[3] = {dim - (dim / 3) * 2, dim / 3, dim / 3};
    L.pyramid = kad_pyramid_project_supported(dim, widths[0], widths[1], widths[2], dtype, H, W) != 0;
    L.partials = L.pyramid;
    for (int i = 0; i < 3; ++i) L.partials = L.partials && kad_lcsa_mask_from_partials_supported(H >> i, W >> i, widths[i]) != 0;
    if (L.partials && kad_pyramid_partial_dims(B, H, W, dim, widths[0], widths[1], widths[2], dtype, &L.nct, &L.nrg) != KAD_OK) L.partials = false;
    if (!L.partials) L.nct = L.nrg = 0;
    size_t o = 0;
    for (int i = 0; i < 3; ++i) {
        const int h = H >> i, w = W >> i, c = widths[i];
        L.path[i] = ((tc_mask >> i) & 1) ? 1 : (kad_dsc_mma_supported(c, c, dtype, h, w) ? 3 : 0);
        L.tiles[i] = kad_dsc_gap_tiles(h, w, c, c, L.path[i]);
        L.ws[i] = plan_branch(o, B, h, w, c, es, L.tiles[i], L.nct, L.nrg);
        o = L.ws[i].end;
    }
    L.bytes = o;
    L.fused_lcsa = L.partials && kad_lcsa_masks3_supported(H, W, widths[0], widths[1], widths[2]) != 0;
    L.tail_prep = L.partials && kad_pyramid_lcsa_supported(dim, widths[0], widths[1], widths[2], dtype, H, W) != 0;
    L.inline_mask = L.tail_prep;
    for (int i = 0; i < 3; ++i)
        L.inline_mask = L.inline_mask && L.path[i] == 3 && kad_dsc_mma_inline_mask_supported(widths[i], widths[i], dtype, H >> i, W >> i) != 0;
    return L;
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" size_t kad_kadconv_workspace_bytes(int B, int H, int W, int dim, int dtype, int tc_branches) {
    if (B <= 0 || H < 4 || W < 4 || dim < 3) return 0;
    return plan_layer(B, H, W, dim, dtype, tc_branches).bytes;
}

// 1 = separate kernels, 2 = first stage in the pyramid tail + mask kernels, 3 = tail + masks inside the deformable convolutions
// 1 = preparation + mask kernel per branch on the branch streams, 2 = first stage in the pyramid tail + mask kernels, 3 = tail +
// masks inside the deformable convolutions, 4 = one launch for the three LCSAs in front of the fork. Default (scheme 0) = 1: it is
// the fastest in every regime measured on the detector forward (CUDA-graph replay, 64 / 8 / 1 images): 1: 15.6 / 4.5 / 3.0 ms,
// 4: 16.0 / 4.9 / 3.4 ms; (earlier build) 1: 16.6 / 4.8 / 3.2, 2: 17.4 / 6.2 / 4.3, 3: 17.3 / 5.9 / 4.2 ms. Fewer launches lose because
// the three branches of a layer are independent until the merge: with one short chain of kernels per branch on its own stream the
// small branches hide behind the full-resolution one, whereas a common kernel in front of the fork (4), a one-block-per-image tail
// (2) or more work inside the largest kernel (3) all lengthen the critical path.
static int resolve_scheme(const LayerPlan& L, bool partials_ok, bool counters, int scheme) {
    if (!partials_ok || scheme <= 1) return 1;
    if (scheme == 4) return L.fused_lcsa ? 4 : 1;
    if (!counters || !L.tail_prep) return 1;
    if (scheme == 3) return L.inline_mask ? 3 : 2;
    return 2;
}

extern "C" int kad_kadconv_launch_count(int B, int H, int W, int dim, int dtype, int tc_branches, int with_counters, int scheme) {
    if (B <= 0 || H < 4 || W < 4 || dim < 3) return 0;
    const LayerPlan L = plan_layer(B, H, W, dim, dtype, tc_branches);
    const int sc = resolve_scheme(L, L.partials, with_counters != 0, scheme);
    int n = L.pyramid ? 1 : 3;
    if (sc == 4) n += 1;
    for (int i = 0; i < 3; ++i) {
        n += (sc == 3 || sc == 4) ? 0 : (sc == 2 ? 1 : (L.partials ? 2 : 4));       // LCSA
        n += L.path[i] == 3 ? 1 : 2;                                    // deformable convolution (+ offset convolution unless fused)
    }
    (void)dtype;
    return n + 1 + 3;      // merge + the three squeeze-excite launches
}

extern "C" int kad_kadconv_forward(const KadLayerArgs* a, void* stream) {
    KAD_CHECK_ARG(a && a->x && a->out && a->workspace && a->status, "kad_kadconv_forward: null pointer");
    KAD_CHECK_ARG(a->B > 0 && a->H >= 4 && a->W >= 4 && a->dim >= 3, "kad_kadconv_forward: bad shape B=%d H=%d W=%d dim=%d", a->B, a->H, a->W, a->dim);
    const int widths[3] = {a->dim - (a->dim / 3) * 2, a->dim / 3, a->dim / 3};
    int tc_mask = 0;
    for (int i = 0; i < 3; ++i) {
        KAD_CHECK_ARG(a->br[i].c == widths[i], "kad_kadconv_forward: branch %d has %d channels, expected %d", i, a->br[i].c, widths[i]);
        if (branch_path(a->br[i], a->dtype, a->H >> i, a->W >> i) == 1) tc_mask |= 1 << i;
    }
    KAD_CHECK_ARG(a->workspace_bytes >= kad_kadconv_workspace_bytes(a->B, a->H, a->W, a->dim, a->dtype, tc_mask),
                  "kad_kadconv_forward: workspace of %zu bytes is too small", a->workspace_bytes);
    KAD_CHECK_ARG((uintptr_t)a->workspace % 256 == 0, "kad_kadconv_forward: workspace must be 256-byte aligned");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: cudaGetDevice: %s", cudaGetErrorString(e));
    KAD_CHECK_ARG(dev >= 0 && dev < MAX_DEVICES, "kad_kadconv_forward: device index %d out of range", dev);
    SideStreams* ss = nullptr;
    int rc = side_streams(dev, &ss);
    if (rc) return rc;
    cudaStream_t main_s = (cudaStream_t)stream;
    cudaStream_t st[3] = {main_s, ss->s[0], ss->s[1]};

    unsigned char* ws = reinterpret_cast<unsigned char*>(a->workspace);
    const LayerPlan L = plan_layer(a->B, a->H, a->W, a->dim, a->dtype, tc_mask);
    // the three pooled projections read the same x: one kernel on the caller's stream, before the branches fork
    const bool pyramid = L.pyramid && (uintptr_t)a->x % 16 == 0;
    const bool partials = pyramid && L.partials;
    const int scheme = resolve_scheme(L, partials, a->counters != nullptr, a->scheme);
    const bool inline_mask = scheme == 3;
    if (scheme == 2 || scheme == 3) {
        KadPyramidArgs q{};
        q.x = a->x; q.B = a->B; q.H = a->H; q.W = a->W; q.dim = a->dim; q.dtype = a->dtype; q.counters = a->counters;
        for (int i = 0; i < 3; ++i) {
            const KadBranchParams& br = a->br[i];
            const int Cp = (br.c + 3) & ~3, w = a->W >> i;
            q.w[i] = br.w_proj; q.bias[i] = br.b_proj; q.t[i] = ws + L.ws[i].t; q.c[i] = br.c;
            q.rowpart[i] = (float*)(ws + L.ws[i].rowpart); q.colpart[i] = (float*)(ws + L.ws[i].colpart);
            q.lcsa_w1[i] = br.lcsa_w1; q.lcsa_b1[i] = br.lcsa_b1; q.lcsa_bn_scale[i] = br.lcsa_bn_scale; q.lcsa_bn_shift[i] = br.lcsa_bn_shift;
            q.lcsa_rowmean[i] = (float*)(ws + L.ws[i].rows);
            q.lcsa_A[i] = (float*)(ws + L.ws[i].scratch); q.lcsa_Sm[i] = (float*)(ws + L.ws[i].scratch) + (size_t)a->B * w * Cp;
        }
        rc = kad_pyramid_project_lcsa(&q, stream);
        if (rc) return rc;
    } else if (pyramid) {
        const float* w3[3] = {a->br[0].w_proj, a->br[1].w_proj, a->br[2].w_proj};
        const float* b3[3] = {a->br[0].b_proj, a->br[1].b_proj, a->br[2].b_proj};
        void* t3[3] = {ws + L.ws[0].t, ws + L.ws[1].t, ws + L.ws[2].t};
        float* rp[3] = {(float*)(ws + L.ws[0].rowpart), (float*)(ws + L.ws[1].rowpart), (float*)(ws + L.ws[2].rowpart)};
        float* cp[3] = {(float*)(ws + L.ws[0].colpart), (float*)(ws + L.ws[1].colpart), (float*)(ws + L.ws[2].colpart)};
        rc = kad_pyramid_project(a->x, w3, b3, t3, a->B, a->H, a->W, a->dim, widths, a->dtype, partials ? rp : nullptr, partials ? cp : nullptr, stream);
        if (rc) return rc;
    }

    if (scheme == 4) {
        // the three LCSAs as one launch in front of the fork
        const float* rp[3]; const float* cp[3]; const float* w1[3]; const float* b1[3]; const float* bm[3]; const float* ba[3];
        const float* w2[3]; const float* b2[3]; const float* w3[3]; const float* b3[3]; void* mk[3];
        for (int i = 0; i < 3; ++i) {
            const KadBranchParams& br = a->br[i];
            rp[i] = (const float*)(ws + L.ws[i].rowpart); cp[i] = (const float*)(ws + L.ws[i].colpart);
            w1[i] = br.lcsa_w1; b1[i] = br.lcsa_b1; bm[i] = br.lcsa_bn_scale; ba[i] = br.lcsa_bn_shift;
            w2[i] = br.lcsa_w2; b2[i] = br.lcsa_b2; w3[i] = br.lcsa_w3; b3[i] = br.lcsa_b3; mk[i] = ws + L.ws[i].mask;
        }
        rc = kad_lcsa_masks3_from_partials(rp, cp, L.nct, L.nrg, w1, b1, bm, ba, w2, b2, w3, b3, mk, a->B, a->H, a->W, widths, 1, a->dtype, stream);
        if (rc) return rc;
    }

    // fork
    if ((e = cudaEventRecord(ss->fork, main_s)) != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: fork: %s", cudaGetErrorString(e));
    for (int i = 1; i < 3; ++i)
        if ((e = cudaStreamWaitEvent(st[i], ss->fork, 0)) != cudaSuccess) return fail(KAD_ERR_CUDA, "kad_kadconv_forward: fork wait: %s", cudaGetErrorString(e));

    KadMergeArgs m{};
    m.x = a->x; m.out = a->out; m.B = a->B; m.H = a->H; m.W = a->W; m.C = a->dim; m.dtype = a->dtype; m.out_cstride = a->out_cstride;
    for (int i = 0; i < 3 && rc == KAD_OK; ++i) {
        const KadBranchParams& br = a->br[i];
        const int h = a->H >> i, w = a->W >> i, c = br.c;
        const int path = L.path[i];
        const int tiles = L.tiles[i];
        const BranchWs p = L.ws[i];
        void* s = (void*)st[i];
        if (!pyramid) {
            rc = kad_pool_project(a->x, br.w_proj, br.b_proj, ws + p.t, a->B, a->H, a->W, a->dim, c, 1 << i, KAD_ACT_NONE, a->dim, c, a->dtype, s);
            if (rc) break;
        }
        if (inline_mask || scheme == 4) {
            // nothing to launch here: the mask is evaluated inside the deformable convolution, or was written in front of the fork
        } else if (scheme == 2) {
            const int Cp = (c + 3) & ~3;
            rc = lcsa_mask_from_prepared((const float*)(ws + p.rows), 1, (const float*)(ws + p.scratch), (const float*)(ws + p.scratch) + (size_t)a->B * w * Cp,
                                         br.lcsa_w2, br.lcsa_b2, br.lcsa_w3, br.lcsa_b3, ws + p.mask, a->B, h, w, c, 1, a->dtype, st[i]);
            if (rc) break;
        } else if (partials) {
            rc = kad_lcsa_mask_from_partials((const float*)(ws + p.rowpart), L.nct, (const float*)(ws + p.colpart), L.nrg,
                                             br.lcsa_w1, br.lcsa_b1, br.lcsa_bn_scale, br.lcsa_bn_shift, br.lcsa_w2, br.lcsa_b2, br.lcsa_w3, br.lcsa_b3,
                                             (float*)(ws + p.scratch), (float*)(ws + p.rows), ws + p.mask, a->B, h, w, c, 1, a->dtype, s);
            if (rc) break;
        } else {
            rc = kad_lcsa_sums(ws + p.t, (float*)(ws + p.rows), (float*)(ws + p.cols), a->B, h, w, c, a->dtype, s);
            if (rc) break;
            rc = kad_lcsa_mask((const float*)(ws + p.rows), (const float*)(ws + p.cols), br.lcsa_w1, br.lcsa_b1, br.lcsa_bn_scale, br.lcsa_bn_shift,
                               br.lcsa_w2, br.lcsa_b2, br.lcsa_w3, br.lcsa_b3, (float*)(ws + p.scratch), ws + p.mask, a->B, h, w, c, 1, a->dtype, s);
            if (rc) break;
        }
        KadDscArgs q{};
        if (path == 3) {
            q.offset_weight = br.w_off; q.offset_bias = br.b_off;       // offsets computed inside the DSC kernel
        } else {
            KadDscArgs d{};
            d.x = ws + p.t; d.weight = br.w_off; d.shift = br.b_off; d.y = ws + p.offset;
            d.B = a->B; d.H = h; d.W = w; d.Cin = c; d.Cout = 18; d.dtype = a->dtype; d.y_f32 = 1; d.act = KAD_ACT_NONE; d.status = a->status;
            d.path = kad_dsc_mma_supported(c, 18, a->dtype, h, w) ? 3 : 0;
            rc = kad_dsc_forward(&d, s);
            if (rc) break;
            q.offset = ws + p.offset; q.offset_f32 = 1;
        }
        q.x = ws + p.t;
        if (inline_mask) {
            const int Cp = (c + 3) & ~3;
            q.lcsa_rowmean = (const float*)(ws + p.rows);
            q.lcsa_A = (const float*)(ws + p.scratch); q.lcsa_Sm = (const float*)(ws + p.scratch) + (size_t)a->B * w * Cp;
            q.lcsa_w2 = br.lcsa_w2; q.lcsa_b2 = br.lcsa_b2; q.lcsa_w3 = br.lcsa_w3; q.lcsa_b3 = br.lcsa_b3;
        } else {
            q.mask = ws + p.mask; q.mask_f32 = 1;
        }
        q.weight = path == 1 ? br.w_dsc_tc : (const void*)br.w_dsc_simt;
        if (path == 3 && !inline_mask) q.mma_frags = br.w_dsc_mma;
        q.scale = br.ep_scale; q.shift = br.ep_shift; q.post = br.ep_post; q.y = ws + p.y; q.gap_partial = (float*)(ws + p.gap);
        q.B = a->B; q.H = h; q.W = w; q.Cin = c; q.Cout = c; q.dtype = a->dtype; q.act = KAD_ACT_RELU; q.path = path; q.status = a->status;
        rc = kad_dsc_forward(&q, s);
        if (rc) break;
        // the channel attention of the branch (squeeze-excite MLP on the sums the DSC kernel wrote) on the branch's own stream:
        // a few microseconds that overlap the other branches; the merge kernel then reads B x c attention values
        rc = kad_se_excite((const float*)(ws + p.gap), tiles, 1.0f / (float)(h * w), br.fc_w1, br.fc_b1, br.fc_w2, br.fc_b2,
                           (float*)(ws + p.att), a->B, c, br.hidden, s);
        if (rc) break;
        m.y[i] = ws + p.y; m.att[i] = (const float*)(ws + p.att); m.c[i] = c; m.h[i] = h; m.w[i] = w;
    }
    // join (always, so that a capture in progress is left well-formed even after an argument error)
    for (int i = 1; i < 3; ++i) {
        cudaError_t e1 = cudaEventRecord(ss->join[i - 1], st[i]);
        cudaError_t e2 = cudaStreamWaitEvent(main_s, ss->join[i - 1], 0);
        if (rc == KAD_OK && (e1 != cudaSuccess || e2 != cudaSuccess))
            rc = fail(KAD_ERR_CUDA, "kad_kadconv_forward: join: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    }
    if (rc) return rc;
    return kad_merge_upsample_residual(&m, stream);
}
