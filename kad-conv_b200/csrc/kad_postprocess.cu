// Batched detection post-processing on the device: per image, best class per anchor, confidence filter, sort by
// confidence, class-aware greedy NMS and the max_det cap, in one kernel launch for the whole batch (one CTA per
// image). Semantics follow non_max_suppression of the reference project (KAD-CNet/utils/general.py:881-990) in
// the configuration its inference scripts use (multi_label off, agnostic off): boxes are shifted by class * max_wh
// so that only boxes of the same class suppress each other; a box is dropped when its IoU with an already kept,
// higher-scoring box exceeds the threshold; ties in score keep the lower anchor index first (deterministic).
#include "kad_common.cuh"

namespace kad {
namespace {

constexpr int NMS_THREADS = 1024;
constexpr int NMS_MAX_ANCHORS = 16384;   // sort buffer in shared memory: 16384 x 8 bytes
constexpr int NMS_CHUNK = 64;
constexpr int NMS_MAX_DET = 1024;
constexpr int NMS_TOP = 4096;            // candidates that are sorted first (the kept boxes nearly always come from these)
constexpr int NMS_TOP_TARGET = 3072;     // how many a chosen threshold should let through
constexpr int NMS_BINS = 4096;           // histogram of 12 key bits

__device__ __forceinline__ bool iou_exceeds(const float4& a, const float4& b, float thr) {
    const float left = fmaxf(a.x, b.x), right = fminf(a.z, b.z), top = fmaxf(a.y, b.y), bottom = fminf(a.w, b.w);
    const float w = fmaxf(right - left, 0.f), h = fmaxf(bottom - top, 0.f);
    const float inter = w * h;
    const float sa = (a.z - a.x) * (a.w - a.y), sb = (b.z - b.x) * (b.w - b.y);
    return inter / (sa + sb - inter) > thr;
}

// pred [B][4+nc][A]; dets [B][max_det][6]; counts [B]
template <typename T>
__global__ void __launch_bounds__(NMS_THREADS, 1)
nms_kernel(const T* __restrict__ pred, int nc, int A, int npow2, float conf_thres, float iou_thres, int max_det, float max_wh,
           float* __restrict__ dets, int* __restrict__ counts) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);          // [npow2] (ordered conf << 32) | ~index
    float4* kept = reinterpret_cast<float4*>(keys + npow2);                              // [max_det] class-shifted boxes
    float4* cbox = kept + max_det;                                                       // [64] shifted boxes of the chunk
    float4* craw = cbox + NMS_CHUNK;                                                     // [64] boxes as reported
    float2* cmeta = reinterpret_cast<float2*>(craw + NMS_CHUNK);                         // [64] (conf, class)
    unsigned long long* cmask = reinterpret_cast<unsigned long long*>(cmeta + NMS_CHUNK);   // [64] intra-chunk suppression
    unsigned int* csupp = reinterpret_cast<unsigned int*>(cmask + NMS_CHUNK);            // [64] suppressed by a kept box
    unsigned char* scls = reinterpret_cast<unsigned char*>(csupp + NMS_CHUNK);          // [npow2] best class of every anchor
    unsigned long long* top = reinterpret_cast<unsigned long long*>(scls + npow2);       // [NMS_TOP] the largest keys (npow2 is a multiple of 64)
    int* hist = reinterpret_cast<int*>(top + NMS_TOP);                                   // [NMS_BINS]
    __shared__ int s_ncand, s_nkept, s_cnt, s_tb, s_above;

    const int b = blockIdx.x, tid = threadIdx.x;
    const T* pb = pred + (size_t)b * (4 + nc) * A;
    // the reference compares scores in the tensor's own type, i.e. against the threshold rounded to that type
    conf_thres = to_f<T>(from_f<T>(conf_thres));
    if (tid == 0) { s_ncand = 0; s_nkept = 0; }
    __syncthreads();

    // 1. best class score per anchor -> sortable key
    int local = 0;
    for (int a = tid; a < npow2; a += NMS_THREADS) {
        unsigned long long key = 0ull;
        if (a < A) {
            // the first maximum wins, as in the reference's argmax over the class scores
            float best = to_f<T>(pb[(size_t)4 * A + a]); int cls = 0;
            for (int c = 1; c < nc; ++c) { const float v = to_f<T>(pb[(size_t)(4 + c) * A + a]); if (v > best) { best = v; cls = c; } }
            scls[a] = (unsigned char)cls;
            if (best > conf_thres) {
                unsigned int u = __float_as_uint(best);
                u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                key = ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)a);
                ++local;
            }
        }
        keys[a] = key;
    }
    if (local) atomicAdd(&s_ncand, local);
    __syncthreads();
    const int ncand = s_ncand;

    // 2. sort, descending. The kept boxes come from the top of the order, so the NMS_TOP largest keys are selected first (all
    // candidates, if there are no more than that; else those above a threshold on the 24 leading key bits, found with two
    // 12-bit histograms), sorted and processed; only if they run out before max_det boxes are kept, the whole array is sorted
    // and the NMS starts over. Either way the boxes are visited in exactly the order of the full sort.
    auto sort_desc = [&](unsigned long long* buf, int n2) {
        for (int k = 2; k <= n2; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < n2; i += NMS_THREADS) {
                    const int ixj = i ^ j;
                    if (ixj > i) {
                        const unsigned long long x = buf[i], y = buf[ixj];
                        const bool desc = (i & k) == 0;
                        if (desc ? (x < y) : (x > y)) { buf[i] = y; buf[ixj] = x; }
                    }
                }
                __syncthreads();
            }
        }
    };
    // 3. greedy NMS over chunks of 64 candidates in score order
    float* out = dets + (size_t)b * max_det * 6;
    auto run_nms = [&](const unsigned long long* buf, int count) {
        for (int c0 = 0; c0 < count; c0 += NMS_CHUNK) {
            if (s_nkept >= max_det) break;
            const int nch = min(NMS_CHUNK, count - c0);
            if (tid < NMS_CHUNK) {
                cmask[tid] = 0ull;
                csupp[tid] = tid < nch ? 0u : 1u;
                if (tid < nch) {
                    const unsigned long long key = buf[c0 + tid];
                    const int a = (int)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull));
                    // box corners are formed in the storage type, as the reference does before it widens to float32
                    const float cx = to_f<T>(pb[a]), cy = to_f<T>(pb[(size_t)A + a]);
                    const float hw = to_f<T>(from_f<T>(to_f<T>(pb[(size_t)2 * A + a]) * 0.5f)), hh = to_f<T>(from_f<T>(to_f<T>(pb[(size_t)3 * A + a]) * 0.5f));
                    float4 r;
                    r.x = to_f<T>(from_f<T>(cx - hw)); r.y = to_f<T>(from_f<T>(cy - hh));
                    r.z = to_f<T>(from_f<T>(cx + hw)); r.w = to_f<T>(from_f<T>(cy + hh));
                    // score and class come from the sort key and the per-anchor table of step 1: no second pass over the class scores
                    const unsigned int u = (unsigned int)(key >> 32);
                    const float best = __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
                    const int cls = scls[a];
                    const float sh = (float)cls * max_wh;
                    craw[tid] = r;
                    cbox[tid] = make_float4(r.x + sh, r.y + sh, r.z + sh, r.w + sh);
                    cmeta[tid] = make_float2(best, (float)cls);
                }
            }
            __syncthreads();
            const int nk = s_nkept;
            for (int p = tid; p < nk * NMS_CHUNK; p += NMS_THREADS) {
                const int k = p / NMS_CHUNK, c = p % NMS_CHUNK;
                if (c < nch && iou_exceeds(kept[k], cbox[c], iou_thres)) atomicOr(&csupp[c], 1u);
            }
            for (int p = tid; p < NMS_CHUNK * NMS_CHUNK; p += NMS_THREADS) {
                const int i = p / NMS_CHUNK, j = p % NMS_CHUNK;
                if (j > i && j < nch && iou_exceeds(cbox[i], cbox[j], iou_thres)) atomicOr(&cmask[i], 1ull << j);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long dead = 0ull;
                int n = nk;
                for (int c = 0; c < nch && n < max_det; ++c) {
                    if (csupp[c] || ((dead >> c) & 1ull)) continue;
                    kept[n] = cbox[c];
                    float* o = out + (size_t)n * 6;
                    o[0] = craw[c].x; o[1] = craw[c].y; o[2] = craw[c].z; o[3] = craw[c].w; o[4] = cmeta[c].x; o[5] = cmeta[c].y;
                    dead |= cmask[c];
                    ++n;
                }
                s_nkept = n;
            }
            __syncthreads();
        }
    };
    // the largest bin t with count(bin >= t) >= target, and how many keys lie in the bins above it (warp 0; 128 bins per lane)
    auto find_bin = [&](int target) {
        if (tid < 32) {
            int seg = 0;
            for (int i = 0; i < NMS_BINS / 32; ++i) seg += hist[tid * (NMS_BINS / 32) + i];
            int suf = seg;                                   // sum over this lane's segment and all higher ones
            for (int d = 1; d < 32; d <<= 1) { const int o = __shfl_down_sync(0xffffffffu, suf, d); if (tid + d < 32) suf += o; }
            const unsigned int reach = __ballot_sync(0xffffffffu, suf >= target);
            const int L = reach ? 31 - __clz(reach) : 0;     // the highest lane whose suffix reaches the target
            if (tid == L) {
                int cum = suf - seg, tb = L * (NMS_BINS / 32);
                for (int bin = (L + 1) * (NMS_BINS / 32) - 1; bin >= L * (NMS_BINS / 32); --bin) {
                    if (cum + hist[bin] >= target) { tb = bin; break; }
                    cum += hist[bin];
                }
                s_tb = tb; s_above = cum;
            }
        }
        __syncthreads();
    };
    bool done = ncand == 0;
    if (!done) {
        // Selection threshold: keys with (key >> sel_shift) >= sel_prefix are taken. It is refined 12 key bits at a time (score bits
        // first, then, among equal scores, the anchor order) until what it lets through fits NMS_TOP: one or two rounds when the
        // scores are spread, more when thousands of anchors share a score.
        unsigned long long sel_prefix = 0ull;
        int sel_shift = 64, above_total = 0, group = ncand;  // keys above the crossing group; size of the crossing group
        for (int shift = 52; above_total + group > NMS_TOP && shift >= 4; shift -= 12) {
            for (int i = tid; i < NMS_BINS; i += NMS_THREADS) hist[i] = 0;
            __syncthreads();
            for (int a = tid; a < npow2; a += NMS_THREADS) {
                const unsigned long long k = keys[a];
                if (k && (sel_shift == 64 || (k >> sel_shift) == sel_prefix)) atomicAdd(&hist[(unsigned int)(k >> shift) & 0xFFFu], 1);
            }
            __syncthreads();
            find_bin(NMS_TOP_TARGET - above_total);
            above_total += s_above;
            group = hist[s_tb];
            sel_prefix = (sel_prefix << 12) | (unsigned long long)s_tb;
            sel_shift = shift;
            __syncthreads();
        }
        if (tid == 0) s_cnt = 0;
        __syncthreads();
        for (int a = tid; a < npow2; a += NMS_THREADS) {
            const unsigned long long k = keys[a];
            if (k && (sel_shift == 64 || (k >> sel_shift) >= sel_prefix)) { const int pos = atomicAdd(&s_cnt, 1); if (pos < NMS_TOP) top[pos] = k; }
        }
        __syncthreads();
        const int M = s_cnt;
        if (M <= NMS_TOP) {
            int n2 = 64;
            while (n2 < M) n2 <<= 1;
            for (int i = M + tid; i < n2; i += NMS_THREADS) top[i] = 0ull;
            __syncthreads();
            sort_desc(top, n2);
            run_nms(top, M);
            done = s_nkept >= max_det || M == ncand;
        }
        if (!done) {                                         // rare: the selection ran out first (or held too many equal prefixes)
            __syncthreads();
            if (tid == 0) s_nkept = 0;
            __syncthreads();
            sort_desc(keys, npow2);
            run_nms(keys, ncand);
        }
    }
    if (tid == 0) counts[b] = s_nkept;
}

// Head decode of one detection scale: raw [B][H][W][4*reg_max + nc] (box distribution logits, then class logits) ->
// columns [a_offset, a_offset + H*W) of pred [B][4 + nc][A]. One thread per (image, cell): the expectation of the
// softmax over each side's reg_max bins gives the distances (left, top, right, bottom) from the cell centre
// (x + 0.5, y + 0.5) in grid units; the box leaves as centre x, centre y, width, height in pixels (times the
// stride), the classes as sigmoid scores. Arithmetic in fp32, one rounding at the store. A thread reads its cell's
// contiguous channels, the stores of a warp are contiguous along the anchor axis.
template <typename T>
__global__ void __launch_bounds__(128)
head_decode_kernel(const T* __restrict__ raw, T* __restrict__ pred, int B, int H, int W, int reg_max, int nc, float stride,
                   int a_offset, int A) {
    const long long cell = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int HW = H * W;
    if (cell >= (long long)B * HW) return;
    const int b = (int)(cell / HW), a = (int)(cell - (long long)b * HW);
    const int y = a / W, x = a - y * W;
    const int no = 4 * reg_max + nc;
    const T* src = raw + cell * no;
    float d[4];
#pragma unroll
    for (int side = 0; side < 4; ++side) {
        const T* v = src + side * reg_max;
        float m = -INFINITY;
        for (int j = 0; j < reg_max; ++j) m = fmaxf(m, to_f<T>(v[j]));
        float den = 0.f, num = 0.f;
        for (int j = 0; j < reg_max; ++j) {
            const float e = __expf(to_f<T>(v[j]) - m);
            den += e; num = fmaf((float)j, e, num);
        }
        d[side] = num / den;
    }
    const float ax = (float)x + 0.5f, ay = (float)y + 0.5f;
    const float x1 = ax - d[0], y1 = ay - d[1], x2 = ax + d[2], y2 = ay + d[3];
    T* dst = pred + (size_t)b * (4 + nc) * A + a_offset + a;
    dst[0] = from_f<T>(0.5f * (x1 + x2) * stride);
    dst[(size_t)A] = from_f<T>(0.5f * (y1 + y2) * stride);
    dst[(size_t)2 * A] = from_f<T>((x2 - x1) * stride);
    dst[(size_t)3 * A] = from_f<T>((y2 - y1) * stride);
    const T* cl = src + 4 * reg_max;
    for (int c = 0; c < nc; ++c) dst[(size_t)(4 + c) * A] = from_f<T>(sigmoidf_(to_f<T>(cl[c])));
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" int kad_nms_max_anchors(void) { return NMS_MAX_ANCHORS; }

extern "C" int kad_nms_batched(const void* pred, int B, int nc, int A, float conf_thres, float iou_thres, int max_det,
                               float max_wh, float* dets, int* counts, int dtype, void* stream) {
    KAD_CHECK_ARG(pred && dets && counts, "kad_nms_batched: null pointer");
    KAD_CHECK_ARG(B > 0 && nc > 0 && A > 0, "kad_nms_batched: bad shape");
    KAD_CHECK_ARG(max_det > 0 && max_det <= NMS_MAX_DET, "kad_nms_batched: max_det must lie in [1, %d]", NMS_MAX_DET);
    KAD_CHECK_ARG(conf_thres >= 0.f && conf_thres <= 1.f && iou_thres >= 0.f && iou_thres <= 1.f, "kad_nms_batched: thresholds must lie in [0, 1]");
    if (A > NMS_MAX_ANCHORS)
        return fail(KAD_ERR_UNSUPPORTED, "kad_nms_batched: %d anchors exceed the %d the in-shared-memory sort holds", A, NMS_MAX_ANCHORS);
    int npow2 = 64;
    while (npow2 < A) npow2 <<= 1;
    KAD_CHECK_ARG(nc <= 256, "kad_nms_batched: at most 256 classes (the per-anchor class table holds bytes)");
    size_t smem = (size_t)npow2 * 8 + (size_t)max_det * 16 + NMS_CHUNK * (16 + 16 + 8 + 8 + 4) + (size_t)npow2 + (size_t)NMS_TOP * 8 + (size_t)NMS_BINS * 4 + 64;
    KAD_DISPATCH_DTYPE(dtype, {
        auto kern = nms_kernel<T>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(KAD_ERR_CUDA, "nms smem attribute: %s", cudaGetErrorString(e));
        kern<<<B, NMS_THREADS, smem, (cudaStream_t)stream>>>((const T*)pred, nc, A, npow2, conf_thres, iou_thres, max_det, max_wh, dets, counts);
    });
    KAD_CHECK_LAUNCH("nms_kernel");
    return KAD_OK;
}

extern "C" int kad_head_decode(const void* raw, void* pred, int B, int H, int W, int reg_max, int nc, float stride,
                               int a_offset, int A, int dtype, void* stream) {
    KAD_CHECK_ARG(raw && pred, "kad_head_decode: null pointer");
    KAD_CHECK_ARG(B > 0 && H > 0 && W > 0 && reg_max > 0 && reg_max <= 64 && nc > 0, "kad_head_decode: bad shape");
    KAD_CHECK_ARG(a_offset >= 0 && (long long)a_offset + (long long)H * W <= A, "kad_head_decode: anchors [%d, %d) outside [0, %d)",
                  a_offset, a_offset + H * W, A);
    const long long cells = (long long)B * H * W;
    KAD_CHECK_ARG((cells + 127) / 128 < (1ll << 31), "kad_head_decode: too many cells");
    KAD_DISPATCH_DTYPE(dtype, {
        head_decode_kernel<T><<<(unsigned)((cells + 127) / 128), 128, 0, (cudaStream_t)stream>>>((const T*)raw, (T*)pred, B, H, W, reg_max, nc,
                                                                                              stride, a_offset, A);
    });
    KAD_CHECK_LAUNCH("head_decode_kernel");
    return KAD_OK;
}
