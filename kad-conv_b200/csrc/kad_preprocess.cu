// Image preprocessing and box post-scaling of the detector's inference script on the device.
//
// letterbox_kernel: cv2.resize(INTER_LINEAR) + cv2.copyMakeBorder + BGR->RGB + HWC->CHW of letterbox()
// (KAD-CNet/utils/augmentations.py:106-136) and KAD-CNet/inference/infer_dior.py:39-46, in one pass over the output, with the
// integer arithmetic OpenCV uses for 8-bit images so that the result equals the CPU path bit for bit: 11-bit fixed-point
// coefficients per output column / row (computed on the host exactly as OpenCV's resize does: rounded (1-f)*2048 and f*2048),
// a horizontal pass in 32-bit integers and the vertical pass ((b0 * (r0 >> 4)) >> 16) + ((b1 * (r1 >> 4)) >> 16) + 2) >> 2.
// A shrink by exactly 2 in both directions takes OpenCV's area path instead (rounded mean of the 2x2 block); mode 1 here.
// The `/255` of the script is not applied here: the detector's first layer takes the uint8 planes (kad_stem_conv_u8).
//
// scale_boxes_kernel: scale_boxes() + clip_boxes() + .round() (KAD-CNet/utils/general.py:824-868, infer_dior.py:56) on the padded
// detections of the batched NMS, float32 arithmetic in the reference's operation order.
#include "kad_common.cuh"

namespace kad {
namespace {

struct LetterboxParams {
    const unsigned char* src;      // [H0][W0][3] BGR
    unsigned char* dst;            // [3][Hn][Wn] RGB planes
    const int* xofs; const short* xa;     // [new_w] left source column, [new_w][2] coefficients
    const int* yofs; const short* yb;     // [new_h] upper source row (may be -1 .. H0-1; clipped here), [new_h][2]
    int H0, W0, Hn, Wn, new_h, new_w, top, left, mode, pad;
};

__global__ void __launch_bounds__(256) letterbox_kernel(const LetterboxParams p) {
    const int x = blockIdx.x * blockDim.x + threadIdx.x, y = blockIdx.y;
    if (x >= p.Wn) return;
    const int rx = x - p.left, ry = y - p.top;
    int v[3] = {p.pad, p.pad, p.pad};
    if (rx >= 0 && rx < p.new_w && ry >= 0 && ry < p.new_h) {
        if (p.mode == 1) {                    // exact 2x shrink: rounded mean of the 2x2 block
            const unsigned char* s0 = p.src + ((size_t)(2 * ry) * p.W0 + 2 * rx) * 3;
            const unsigned char* s1 = s0 + (size_t)p.W0 * 3;
#pragma unroll
            for (int c = 0; c < 3; ++c) v[c] = (s0[c] + s0[3 + c] + s1[c] + s1[3 + c] + 2) >> 2;
        } else {
            const int x0 = p.xofs[rx], x1 = min(x0 + 1, p.W0 - 1);
            const int a0 = p.xa[2 * rx], a1 = p.xa[2 * rx + 1];
            const int sy = p.yofs[ry], y0 = min(max(sy, 0), p.H0 - 1), y1 = min(max(sy + 1, 0), p.H0 - 1);
            const int b0 = p.yb[2 * ry], b1 = p.yb[2 * ry + 1];
            const unsigned char* r0 = p.src + (size_t)y0 * p.W0 * 3;
            const unsigned char* r1 = p.src + (size_t)y1 * p.W0 * 3;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const int h0 = r0[x0 * 3 + c] * a0 + r0[x1 * 3 + c] * a1;
                const int h1 = r1[x0 * 3 + c] * a0 + r1[x1 * 3 + c] * a1;
                v[c] = (((b0 * (h0 >> 4)) >> 16) + ((b1 * (h1 >> 4)) >> 16) + 2) >> 2;
            }
        }
    }
    const size_t plane = (size_t)p.Hn * p.Wn, o = (size_t)y * p.Wn + x;
    p.dst[o] = (unsigned char)v[2];                  // R
    p.dst[plane + o] = (unsigned char)v[1];          // G
    p.dst[2 * plane + o] = (unsigned char)v[0];      // B
}

// dets [B][max_det][6]; geom [B][5] = gain, pad_x, pad_y, width0, height0 (float32, one row per image)
__global__ void scale_boxes_kernel(float* __restrict__ dets, const int* __restrict__ counts, const float* __restrict__ geom, int max_det, int do_round) {
    const int b = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= counts[b] || i >= max_det) return;
    const float gain = geom[5 * b], px = geom[5 * b + 1], py = geom[5 * b + 2], w0 = geom[5 * b + 3], h0 = geom[5 * b + 4];
    float* d = dets + ((size_t)b * max_det + i) * 6;
    float x1 = (d[0] - px) / gain, y1 = (d[1] - py) / gain, x2 = (d[2] - px) / gain, y2 = (d[3] - py) / gain;
    x1 = fminf(fmaxf(x1, 0.f), w0); x2 = fminf(fmaxf(x2, 0.f), w0);
    y1 = fminf(fmaxf(y1, 0.f), h0); y2 = fminf(fmaxf(y2, 0.f), h0);
    if (do_round) { x1 = rintf(x1); y1 = rintf(y1); x2 = rintf(x2); y2 = rintf(y2); }
    d[0] = x1; d[1] = y1; d[2] = x2; d[3] = y2;
}

}  // namespace
}  // namespace kad

using namespace kad;

extern "C" int kad_letterbox_u8(const void* src_bgr_hwc, void* dst_rgb_chw, int H0, int W0, int Hn, int Wn,
                                int new_h, int new_w, int top, int left, int area2x,
                                const int* xofs, const short* xalpha, const int* yofs, const short* ybeta,
                                int pad_value, void* stream) {
    KAD_CHECK_ARG(src_bgr_hwc && dst_rgb_chw, "kad_letterbox_u8: null pointer");
    KAD_CHECK_ARG(H0 > 0 && W0 > 0 && Hn > 0 && Wn > 0 && new_h > 0 && new_w > 0 && Hn <= 65535, "kad_letterbox_u8: bad shape");
    KAD_CHECK_ARG(top >= 0 && left >= 0 && top + new_h <= Hn && left + new_w <= Wn, "kad_letterbox_u8: the resized image (%d x %d at %d, %d) does not fit the %d x %d output",
                  new_w, new_h, left, top, Wn, Hn);
    KAD_CHECK_ARG(area2x ? (H0 == 2 * new_h && W0 == 2 * new_w) : (xofs && xalpha && yofs && ybeta), "kad_letterbox_u8: missing coefficient tables");
    KAD_CHECK_ARG(pad_value >= 0 && pad_value <= 255, "kad_letterbox_u8: pad value out of range");
    LetterboxParams p{};
    p.src = (const unsigned char*)src_bgr_hwc; p.dst = (unsigned char*)dst_rgb_chw;
    p.xofs = xofs; p.xa = xalpha; p.yofs = yofs; p.yb = ybeta;
    p.H0 = H0; p.W0 = W0; p.Hn = Hn; p.Wn = Wn; p.new_h = new_h; p.new_w = new_w; p.top = top; p.left = left; p.mode = area2x ? 1 : 0; p.pad = pad_value;
    letterbox_kernel<<<dim3((Wn + 255) / 256, Hn), 256, 0, (cudaStream_t)stream>>>(p);
    KAD_CHECK_LAUNCH("letterbox_kernel");
    return KAD_OK;
}

extern "C" int kad_scale_boxes(float* dets, const int* counts, const float* geom, int B, int max_det, int do_round, void* stream) {
    KAD_CHECK_ARG(dets && counts && geom, "kad_scale_boxes: null pointer");
    KAD_CHECK_ARG(B > 0 && B <= 65535 && max_det > 0, "kad_scale_boxes: bad shape");
    scale_boxes_kernel<<<dim3((max_det + 127) / 128, B), 128, 0, (cudaStream_t)stream>>>(dets, counts, geom, max_det, do_round);
    KAD_CHECK_LAUNCH("scale_boxes_kernel");
    return KAD_OK;
}
