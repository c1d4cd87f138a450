/*
 * Plain-C restatement of the modulated deformable 3x3 convolution (DCNv2) on the KAD-Conv hot path.
 *
 * TEST INFRASTRUCTURE ONLY: built by oracle/Makefile into oracle/_build/, loaded by the tests as a second,
 * independent checker next to oracle/kad_oracle.py. Nothing in the shipped package links or loads it.
 *
 * Follows the sampling rule the reference restates in
 * KAD-CNet/inference/acceleration/kadc_dcn_direct.py:49-107 (== torchvision.ops.deform_conv2d as called at
 * KAD-Conv/kadconv/kad_conv.py:66-67): offset channel 2k = dy, 2k+1 = dx of tap k = ky*3+kx; a sample counts
 * only if -1 < y < H and -1 < x < W; each corner counts only inside the image; value x mask; stride 1, pad 1.
 * Layout NCHW, float32 storage, double accumulation. Parity: pinned by tests/golden/dcn_op.npz.
 */
#include <math.h>
#include <stddef.h>

void kad_oracle_deform_conv3x3(const float* x, const float* offset, const float* mask, const float* weight,
                               const float* bias, float* y, int B, int Cin, int Cout, int H, int W) {
    const size_t HW = (size_t)H * W;
    for (int b = 0; b < B; ++b) {
        for (int py = 0; py < H; ++py) {
            for (int px = 0; px < W; ++px) {
                const size_t pix = (size_t)py * W + px;
                for (int o = 0; o < Cout; ++o) {
                    double acc = bias ? (double)bias[o] : 0.0;
                    for (int k = 0; k < 9; ++k) {
                        const float dy = offset ? offset[((size_t)b * 18 + 2 * k) * HW + pix] : 0.f;
                        const float dx = offset ? offset[((size_t)b * 18 + 2 * k + 1) * HW + pix] : 0.f;
                        const float m = mask ? mask[((size_t)b * 9 + k) * HW + pix] : 1.f;
                        const float sy = (float)(py + k / 3 - 1) + dy, sx = (float)(px + k % 3 - 1) + dx;
                        if (!(sy > -1.f && sy < (float)H && sx > -1.f && sx < (float)W)) continue;
                        const int y0 = (int)floorf(sy), x0 = (int)floorf(sx);
                        const float ly = sy - (float)y0, lx = sx - (float)x0;
                        const float w00 = (1.f - ly) * (1.f - lx), w01 = (1.f - ly) * lx, w10 = ly * (1.f - lx), w11 = ly * lx;
                        for (int i = 0; i < Cin; ++i) {
                            const float* xc = x + ((size_t)b * Cin + i) * HW;
                            float v = 0.f;
                            if (y0 >= 0 && x0 >= 0) v += w00 * xc[(size_t)y0 * W + x0];
                            if (y0 >= 0 && x0 + 1 < W) v += w01 * xc[(size_t)y0 * W + x0 + 1];
                            if (y0 + 1 < H && x0 >= 0) v += w10 * xc[(size_t)(y0 + 1) * W + x0];
                            if (y0 + 1 < H && x0 + 1 < W) v += w11 * xc[(size_t)(y0 + 1) * W + x0 + 1];
                            acc += (double)weight[(((size_t)o * Cin + i) * 9) + k] * (double)(v * m);
                        }
                    }
                    y[((size_t)b * Cout + o) * HW + pix] = (float)acc;
                }
            }
        }
    }
}
