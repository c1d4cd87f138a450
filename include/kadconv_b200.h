/*
 * kadconv_b200 -- C ABI of the B200 (sm_100a) KAD-Conv inference kernels.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless the name says host;
 *   - activations are NHWC ("channels last"): element (b, y, x, c) of a [B,H,W,C] tensor lives at
 *     ((b*H + y)*W + x)*C + c; parameters are float32 unless stated otherwise;
 *   - `dtype` is the storage type of the activations (KAD_F32 / KAD_F16 / KAD_BF16); all arithmetic
 *     accumulates in float32;
 *   - the caller owns every buffer (inputs, outputs, scratch); nothing is allocated, nothing
 *     synchronises, every kernel is launched on `stream` (a cudaStream_t passed as void*) and the
 *     calls can be captured in a CUDA graph;
 *   - most kernels are launched with programmatic stream serialization: they read their PARAMETERS (weights,
 *     bias, scale / shift vectors) first, then wait for everything in front of them in the stream, then touch
 *     activations. Activations may come from any earlier work in the stream; parameters must not be written by
 *     the kernel that IMMEDIATELY precedes the call in the same stream (anything in between, or one
 *     synchronisation after the weights were prepared, is enough);
 *   - return value 0 on success, a negative KAD_ERR_* otherwise; kad_last_error_string() gives the
 *     reason for the calling thread. No call throws or exits.
 *
 * Each declaration names the reference interface it stands in for (paths relative to the
 * reference project). The reference's own native ABI is a pair of pybind11 torch extensions taking
 * torch::Tensor (KAD-CNet/inference/acceleration/kadc_dcn16.cpp:247-330 and kadc_gemm_silu.cpp:22-33).
 */
#ifndef KADCONV_B200_H_
#define KADCONV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { KAD_F32 = 0, KAD_F16 = 1, KAD_BF16 = 2 };
enum { KAD_OK = 0, KAD_ERR_INVALID = -1, KAD_ERR_CUDA = -2, KAD_ERR_UNSUPPORTED = -3, KAD_ERR_DEVICE_WAIT = -4 };
enum { KAD_ACT_NONE = 0, KAD_ACT_SILU = 1, KAD_ACT_RELU = 2 };

/* Library version (major*10000 + minor*100 + patch). */
int kad_version(void);
/* sizeof of an argument struct of this header as the library was compiled: 0 KadDscArgs, 1 KadPyramidArgs, 2 KadMergeArgs,
 * 3 KadBranchParams, 4 KadLayerArgs (-1 otherwise). A binding in another language checks its own declarations against it: the
 * library reads every field, so a struct declared too short is read past its end. */
int kad_struct_size(int which);
/* Reason for the last non-zero return on this thread (empty string if none). */
const char* kad_last_error_string(void);

/* Layout conversion at the module boundary: the reference is NCHW-contiguous end to end
 * (KAD-Conv/kadconv/fast.py:38-40 requires is_contiguous()). */
int kad_nchw_to_nhwc(const void* src, void* dst, int B, int C, int H, int W, int dtype, void* stream);
int kad_nhwc_to_nchw(const void* src, void* dst, int B, int C, int H, int W, int dtype, void* stream);

/* Modulated deformable 3x3 convolution, stride 1, padding 1, with a fused per-channel epilogue.
 *   y[b,p,o] = post[o] * act( scale[o] * sum_{k,i} Wt[k][i][o] * m[b,p,k] * bilinear(x[b,:,:,i], p + k + d[b,p,k]) + shift[o] )
 * Replaces torchvision.ops.deform_conv2d as called by DSC.forward (KAD-Conv/kadconv/kad_conv.py:63-67,
 * KAD-CNet/models/module/ops.py:68-72) together with the BatchNorm, ReLU and branch scale that follow it
 * in KADConv (kad_conv.py:101-102,:110); native counterpart: dcn16x32_kernel
 * (KAD-CNet/inference/acceleration/kadc_dcn16_kernel.cu:92-314).
 *
 *   x       [B,H,W,Cin]  dtype
 *   offset  [B,H,W,18]   float32 if offset_f32 else dtype; channel 2k = dy, 2k+1 = dx of tap k = ky*3+kx.
 *                        NULL means zero offsets (an ordinary 3x3 convolution).
 *   mask    [B,H,W,9]    same type rule as offset (mask_f32); NULL means all ones.
 *   weight  SIMT path:   float32 [9][Cin][Cout]  (tap-major, Cout contiguous), packed by kad_dsc_pack_weight_simt()
 *           tensor path: see kad_dsc_tc_supported(); dtype, packed by kad_dsc_pack_weight_tc()
 *   scale/shift/post     float32 [Cout] or NULL (1 / 0 / 1). Conv bias goes into shift.
 *   act     KAD_ACT_*
 *   y       [B,H,W,Cout] float32 if y_f32 else dtype
 *   gap_partial  NULL, or float32 [B][gap_tiles][Cout]: per-tile sums of y over pixels, in a fixed order
 *                (deterministic); gap_tiles = kad_dsc_gap_tiles(H, W, Cin, Cout, path).
 */
typedef struct KadDscArgs {
    const void* x; const void* offset; const void* mask; const void* weight;
    const float* scale; const float* shift; const float* post;
    void* y; float* gap_partial;
    int B, H, W, Cin, Cout;
    int dtype, offset_f32, mask_f32, y_f32, act;
    int path;            /* 0 = SIMT (any shape, any dtype); 1 = tcgen05 implicit GEMM (see kad_dsc_tc_supported);
                            2 = the same on CTA pairs (tcgen05 cta_group::2, cluster of 2; needs Cout % 32 == 0);
                            3 = warp-level tensor-core kernel for small channel counts (see kad_dsc_mma_supported):
                                weight in the SIMT layout, operands rounded to dtype, float32 accumulation */
    int* status;         /* device int[4], zeroed by the caller; the tensor path records a wait that gave up here */
    /* path 3 only, optional: weights of the offset convolution (float32 [9][Cin][18], kad_dsc_pack_weight_simt of
       DSC.conv_offset.weight) and its bias (float32 [18] or NULL). When offset_weight is set, `offset` is ignored and
       the kernel computes the offsets of its own pixels itself (kad_conv.py:64 fused into :66-67): the offset
       tensor is never written to memory. */
    const float* offset_weight; const float* offset_bias;
    /* path 3 with offset_weight only, optional: the modulation mask of LCSA.forward + sigmoid (kad_conv.py:24-39,:65) evaluated
       inside the kernel, per pixel, so that the mask tensor is never written to memory. When lcsa_rowmean is set, `mask` is
       ignored. With C = Cin and Cp = C rounded up to a multiple of 4:
         lcsa_rowmean float32 [B][H][C] means of x over the row (pool_h)
         lcsa_A      float32 [B][W][Cp] and lcsa_Sm float32 [W][Cp]: the separable 1x11 + BatchNorm stage per column, as
                     kad_pyramid_project_lcsa / kad_lcsa_mask_from_partials compute them (16-byte aligned)
         lcsa_w2 [C][11], lcsa_b2 [C] (11x1 depthwise), lcsa_w3 [9][C], lcsa_b3 [9] (1x1)
       kad_dsc_mma_inline_mask_supported() says whether the operands fit shared memory for this shape. */
    const float* lcsa_rowmean; const float* lcsa_A; const float* lcsa_Sm;
    const float* lcsa_w2; const float* lcsa_b2; const float* lcsa_w3; const float* lcsa_b3;
    /* path 3 with offset_weight and a mask tensor, optional: the weight fragments of both convolutions as kad_dsc_mma_pack_frags
       wrote them (kad_dsc_mma_frag_bytes bytes, 16-byte aligned). Every block then copies them instead of deriving them from
       `weight` and `offset_weight`, which must still be passed (they are what the fragments were packed from). */
    const void* mma_frags;
} KadDscArgs;
int kad_dsc_forward(const KadDscArgs* args, void* stream);
int kad_dsc_gap_tiles(int H, int W, int Cin, int Cout, int path);
/* 1 if the tcgen05 path can run this shape: dtype f16/bf16, Cin % 32 == 0, Cout % 16 == 0, Cout <= 256. */
int kad_dsc_tc_supported(int Cin, int Cout, int dtype);
/* 1 if path 3 can run this shape: dtype f16/bf16, 4 <= Cin <= 64, Cout <= 64, and the image rows a group of 256
 * pixels touches (W * Cin * 2 bytes each) fit in shared memory beside the kernel's tables. x must be 16-byte aligned.
 * Path 3 writes its channel sums per group of 256 pixels: kad_dsc_gap_tiles(..., 3) = ceil(H*W / 256). */
int kad_dsc_mma_supported(int Cin, int Cout, int dtype, int H, int W);
int kad_dsc_mma_inline_mask_supported(int Cin, int Cout, int dtype, int H, int W);
size_t kad_dsc_mma_frag_bytes(int Cin, int Cout, int dtype);
int kad_dsc_mma_pack_frags(const float* weight_simt, const float* offset_weight_simt, void* dst, int Cin, int Cout, int dtype, void* stream);
/* Packs W[Cout][Cin][3][3] (float32, the layout of DSC.weight) into the tensor path's K-major
 * operand: dst is dtype [9*Cin/64 (rounded up)][Cout][64]; K index = (ci/32)*288 + tap*32 + ci%32. */
int kad_dsc_pack_weight_tc(const float* w_oihw, void* dst, int Cin, int Cout, int dtype, void* stream);
size_t kad_dsc_packed_weight_bytes(int Cin, int Cout, int dtype);
/* Packs W[Cout][Cin][3][3] (float32) into the SIMT path's float32 [9][Cin][Cout]. The same routine packs
 * DSC.conv_offset.weight ([18][Cin][3][3]) for the offset convolution, which runs as kad_dsc_forward
 * with offset = mask = NULL (KAD-Conv/kadconv/kad_conv.py:55-56,:64). */
int kad_dsc_pack_weight_simt(const float* w_oihw, float* dst, int Cin, int Cout, void* stream);

/* Average pool (kernel = stride = pool, floor mode) fused with a 1x1 convolution, bias and activation:
 *   y[b,q,o] = act( sum_i w[o][i] * mean_{p in pool x pool block q} x[b,p,i] + bias[o] )
 * Replaces F.avg_pool2d + convs[i][0] in KADConv.forward (kad_conv.py:115,:101) and, with pool = 1 and
 * KAD_ACT_SILU, Conv.forward_fuse for k = 1 (KAD-CNet/models/common.py:56-57); native counterpart:
 * gemm_bias_silu_kernel (KAD-CNet/inference/acceleration/kadc_gemm_silu.cu:125-176).
 *   x [B,H,W,Cin] dtype (channel stride x_cstride >= Cin elements per pixel, so a channel slice of a wider
 *   tensor can be read in place), w float32 [Cout][Cin], bias float32 [Cout] or NULL,
 *   y [B,H/pool,W/pool,Cout] dtype written with per-pixel stride y_cstride >= Cout (concat in place). */
int kad_pool_project(const void* x, const float* w, const float* bias, void* y,
                     int B, int H, int W, int Cin, int Cout, int pool, int act,
                     int x_cstride, int y_cstride, int dtype, void* stream);

/* The whole branch pyramid of a KAD-Conv layer in one pass over x: t[i] = conv1x1_i(avg_pool2d(x, 2^i)) + bias_i, i = 0..2
 * (KADConv.forward, kad_conv.py:115 with convs[i][0], :101): three calls of kad_pool_project that share their input.
 *   x [B,H,W,dim] dtype; w[i] float32 [c[i]][dim], bias[i] float32 [c[i]] or NULL; t[i] [B,H>>i,W>>i,c[i]] dtype.
 * Operands are rounded to dtype (the pooled means as well, as F.avg_pool2d rounds them), accumulation is float32.
 * kad_pyramid_project_supported: dtype f16/bf16, dim % 8 == 0, widths <= 64, H, W >= 4, a 4-row tile fits shared memory. */
int kad_pyramid_project_supported(int dim, int c0, int c1, int c2, int dtype, int H, int W);
/* Optional by-products (both or neither; NULL to skip) for the LCSA that follows, whose pool_h / pool_w (kad_conv.py:27-28)
 * are sums over the very tensors this kernel writes: rowpart[i] float32 [B][H>>i][n_col_tiles][c[i]] (sum over the columns
 * of one tile) and colpart[i] float32 [B][n_row_groups][W>>i][c[i]] (sum over the rows one block covers), of the values as
 * stored; (n_col_tiles, n_row_groups) from kad_pyramid_partial_dims. kad_lcsa_mask_from_partials consumes them. */
int kad_pyramid_partial_dims(int B, int H, int W, int dim, int c0, int c1, int c2, int dtype, int* n_col_tiles, int* n_row_groups);
int kad_pyramid_project(const void* x, const float* const* w, const float* const* bias, void* const* t,
                        int B, int H, int W, int dim, const int* c, int dtype,
                        float* const* rowpart, float* const* colpart, void* stream);
/* kad_pyramid_project that also finishes the first, separable stage of the three LCSAs (kad_conv.py:27-31: pool_h + pool_w,
 * the 1x11 depthwise convolution, BatchNorm) in the tail of the same kernel: the block that finishes an image last reduces
 * that image's partial sums (fixed order, so the result does not depend on which block it is) and writes, per branch i,
 *   lcsa_rowmean[i] float32 [B][h_i][c_i] (means over the row), lcsa_A[i] float32 [B][w_i][Cp_i], lcsa_Sm[i] float32 [w_i][Cp_i]  (Cp = c rounded up to 4)
 * which kad_dsc_forward (path 3, lcsa_* fields) consumes; the same values kad_lcsa_mask_from_partials derives in a kernel of
 * its own. lcsa_w1[i] [c_i][11], lcsa_b1[i] [c_i]: the 1x11 depthwise convolution; lcsa_bn_scale / lcsa_bn_shift [c_i]: folded BatchNorm.
 * counters: device int[B], zero before the first call; every call leaves them zero again (calls that share them must not overlap).
 * kad_pyramid_lcsa_supported: kad_pyramid_project_supported, the widest column-sum table (W * c0 floats) fits the block's shared memory,
 * and this variant's kernel partitions the partial sums as kad_pyramid_partial_dims says (true for maps up to 128 columns whose
 * 4-row tile of x fits shared memory in one piece; wider or deeper inputs get 0 and take kad_pyramid_project + kad_lcsa_mask_from_partials). */
typedef struct KadPyramidArgs {
    const void* x; const float* w[3]; const float* bias[3]; void* t[3];
    int B, H, W, dim, c[3], dtype;
    float* rowpart[3]; float* colpart[3];
    int* counters;
    const float* lcsa_w1[3]; const float* lcsa_b1[3]; const float* lcsa_bn_scale[3]; const float* lcsa_bn_shift[3];
    float* lcsa_rowmean[3]; float* lcsa_A[3]; float* lcsa_Sm[3];
} KadPyramidArgs;
int kad_pyramid_lcsa_supported(int dim, int c0, int c1, int c2, int dtype, int H, int W);
int kad_pyramid_project_lcsa(const KadPyramidArgs* args, void* stream);

/* Average pool, kernel = stride = pool, floor mode, NHWC: F.avg_pool2d as used for the branch pyramid
 * (KAD-Conv/kadconv/kad_conv.py:115) when the pooled tensor feeds the tensor-core 1x1 GEMM. */
int kad_avg_pool(const void* x, void* y, int B, int H, int W, int C, int pool, int dtype, void* stream);

/* Detector glue (KAD-CNet-S outside its KAD-Conv layers), NHWC:
 *  kad_avg_pool2x2s1    avg_pool2d(x, 2, 1, 0) of AConv.forward (KAD-CNet/models/common.py:65-66): [B,H,W,C] -> [B,H-1,W-1,C]
 *  kad_bias_act_inplace y = act(y + bias[c]) on [M][C]: the bias + SiLU of Conv.forward_fuse (common.py:56-57) after a
 *                       bias-free 3x3 convolution (counterpart of bias_silu_float4_kernel, kadc_gemm_silu.cu:67-88)
 *  kad_image_to_nhwc    uint8 [B,C,H,W] image batch -> dtype [B,H,W,Cp], value * scale, channels C..Cp-1 zero: the
 *                       `/255` normalisation of KAD-CNet/inference/infer_dior.py:39-46 fused with the layout change */
int kad_avg_pool2x2s1(const void* x, void* y, int B, int H, int W, int C, int dtype, void* stream);
/* The detector's first layer on raw images, in one kernel: uint8 [B,Cin,H,W] -> 3x3 convolution with stride 2 and
 * padding 1 -> * scale + bias -> activation -> [B,(H-1)/2+1,(W-1)/2+1,Cout] dtype (NHWC). Replaces the `/255`
 * of KAD-CNet/inference/infer_dior.py:39-46 followed by Conv.forward_fuse of layer 0 (KAD-CNet/models/common.py:56-57;
 * yaml: [-1, 1, Conv, [32, 3, 2]]). w float32 [Cout][Cin][3][3] (BatchNorm folded), bias float32 [Cout] or NULL.
 * kad_stem_conv_supported: dtype f16/bf16, Cin <= 4, Cout % 8 == 0, Cout <= 64. */
int kad_stem_conv_supported(int Cin, int Cout, int dtype);
int kad_stem_conv_u8(const void* img_u8, const float* w_oihw, const float* bias, void* y,
                     int B, int Cin, int H, int W, int Cout, float scale, int act, int dtype, void* stream);
int kad_bias_act_inplace(void* y, const float* bias, long long M, int C, int act, int dtype, void* stream);
/* The same out of place: out[m][0..C) = act(y[m][0..C) + bias) with out rows out_cstride (0 = C) elements apart, so the
 * result of a convolution lands in its channel slice of a concatenation (the torch.cat of ELAN1.forward /
 * RepNCSPELAN4.forward, KAD-CNet/models/common.py) without a copy of its own. */
int kad_bias_act_to(const void* y, const float* bias, void* out, long long M, int C, int out_cstride, int act, int dtype, void* stream);
/* Copy of a channel slice between NHWC tensors of different widths: dst[m][dst_coff .. dst_coff + C) = src[m][src_coff .. src_coff + C)
 * for m < M, rows src_cstride / dst_cstride elements apart. The `chunk(2, 1)` of ELAN1.forward (KAD-CNet/models/common.py) feeds a
 * library 3x3 convolution, which wants a dense tensor, and the convolution's output goes back into the concatenation: both moves
 * are this call (the widest vectors that the addresses allow) instead of a strided tensor copy. dtype: any KAD_* (2 or 4 bytes). */
int kad_copy_channels(const void* src, int src_cstride, int src_coff, void* dst, int dst_cstride, int dst_coff,
                      long long M, int C, int dtype, void* stream);
/* nn.Upsample(scale_factor=2, mode='nearest') followed by Concat([upsampled, skip]) (the top-down path of the neck,
 * yaml: [-1, 1, nn.Upsample, [None, 2, 'nearest']], [[-1, k], 1, Concat, [1]]) in one pass:
 *   low [B,h,w,C1], skip [B,2h,2w,C2] -> out [B,2h,2w,C1+C2], all NHWC dtype. */
int kad_upsample2x_concat(const void* low, const void* skip, void* out, int B, int h, int w, int C1, int C2, int dtype, void* stream);
int kad_image_to_nhwc(const void* img_u8, void* y, int B, int C, int H, int W, int Cp, float scale, int dtype, void* stream);

/* LCSA, step 1: row sums [B,H,C] (over x) and column sums [B,W,C] (over y) of x[B,H,W,C], float32.
 * Replaces pool_h / pool_w of LCSA.forward (kad_conv.py:27-28,:39). */
int kad_lcsa_sums(const void* x, float* rowsum, float* colsum, int B, int H, int W, int C, int dtype, void* stream);
/* LCSA, step 2: mask = sigmoid(1x1( dw11x1( relu(bn(dw1x11(rowmean + colmean))) ) )), [B,H,W,9].
 * Replaces LCSA.excite + the sigmoid in DSC.forward (kad_conv.py:29-39,:65); counterpart of the Triton
 * kernels k_reduce_hconv_bn_relu / k_vconv_pointwise9 (kadc_fused_sm75.py:830-888,:905-996).
 *   w1 [C][11] (1x11 depthwise), b1 [C], bn_scale/bn_shift [C] (folded BatchNorm), w2 [C][11] (11x1),
 *   b2 [C], w3 [9][C], b3 [9]; scratch float32 [B*W*C + W*C]; mask float32 if mask_f32 else dtype. */
int kad_lcsa_mask(const float* rowsum, const float* colsum,
                  const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                  const float* w2, const float* b2, const float* w3, const float* b3,
                  float* scratch, void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream);

/* LCSA steps 1 + 2 from the partial sums of kad_pyramid_project (no second pass over the branch tensor): the sums over
 * tiles are finished here (rowsum float32 [B][H][C] is written as a by-product), then the mask as in kad_lcsa_mask.
 * Works on 128 consecutive pixels per block, so narrow feature maps keep their lanes busy. scratch: float32
 * [(B + 1) * W * Cp] with Cp = C rounded up to a multiple of 4, 16-byte aligned.
 * kad_lcsa_mask_from_partials_supported: C <= 256 and the per-row operands fit shared memory. */
int kad_lcsa_mask_from_partials_supported(int H, int W, int C);
int kad_lcsa_mask_from_partials(const float* rowpart, int n_col_tiles, const float* colpart, int n_row_groups,
                                const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                                const float* w2, const float* b2, const float* w3, const float* b3,
                                float* scratch, float* rowsum, void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream);

/* The LCSA masks of the three branches of a KAD-Conv layer in ONE launch, from the partial sums of kad_pyramid_project: what three
 * calls of kad_lcsa_mask_from_partials compute (bit-identical), with the first stage recomputed per block in shared memory
 * instead of passing through a preparation kernel and a scratch buffer. Arrays of three (branch i works at (H >> i) x (W >> i)
 * with c[i] channels); rowpart / colpart and their tile counts as kad_pyramid_project wrote them; mask[i] [B][H>>i][W>>i][9].
 * kad_lcsa_masks3_supported: W <= 128 (a block spans all columns of its rows) and the per-image operands fit shared memory. */
int kad_lcsa_masks3_supported(int H, int W, int c0, int c1, int c2);
int kad_lcsa_masks3_from_partials(const float* const* rowpart, const float* const* colpart, int n_col_tiles, int n_row_groups,
                                  const float* const* w1, const float* const* b1, const float* const* bn_scale, const float* const* bn_shift,
                                  const float* const* w2, const float* const* b2, const float* const* w3, const float* const* b3,
                                  void* const* mask, int B, int H, int W, const int* c, int mask_f32, int dtype, void* stream);

/* LCSA step 2 without a scratch argument and without any allocation. No counterpart in the reference project: it
 * exists for hosts that cannot create device memory where they call this library (a server whose own pool took all
 * of HBM at start-up, or a frame loop that must avoid the device-wide synchronisation of cudaMalloc / cudaFree).
 * The scratch kad_lcsa_mask() asks for lives in a fixed array inside the library's device image instead
 * (kad_lcsa_mask_noalloc_max_floats() float32 values, 4 MiB, held by every GPU that loads the library until the
 * process exits). Same arguments and result as kad_lcsa_mask minus `scratch`.
 *   - (B+1)*W*C must not exceed kad_lcsa_mask_noalloc_max_floats(); larger problems get KAD_ERR_UNSUPPORTED.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call during start-up, before any stream capture begins on that device.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different streams) race on it.
 *     Nothing needs clearing between calls; each call overwrites the part it reads. */
size_t kad_lcsa_mask_noalloc_max_floats(void);
int kad_lcsa_mask_noalloc(const float* rowsum, const float* colsum,
                          const float* w1, const float* b1, const float* bn_scale, const float* bn_shift,
                          const float* w2, const float* b2, const float* w3, const float* b3,
                          void* mask, int B, int H, int W, int C, int mask_f32, int dtype, void* stream);

/* SE excite from the DSC epilogue's per-tile sums: att[b,:] = sigmoid(W2 relu(W1 mean + b1) + b2).
 * Replaces y.mean((2,3)) and fc[i] in KADConv.forward (kad_conv.py:105-109,:117); native counterpart:
 * partial_gap_se_kernel (kadc_dcn16_kernel.cu:499-556).
 *   gap_partial [B][tiles][C], w1 [Hd][C], b1 [Hd], w2 [C][Hd], b2 [C], att float32 [B][C]. */
int kad_se_excite(const float* gap_partial, int tiles, float inv_count,
                  const float* w1, const float* b1, const float* w2, const float* b2,
                  float* att, int B, int C, int Hd, void* stream);

/* Channel attention on a full tensor (squeeze + rescale), for SE blocks outside KAD-Conv:
 * kad_se_squeeze writes float32 partial sums [B][tiles][C] (tiles = kad_se_squeeze_tiles(H,W));
 * kad_se_rescale computes y = x * att[b,c]. */
int kad_se_squeeze_tiles(int H, int W);
int kad_se_squeeze(const void* x, float* gap_partial, int B, int H, int W, int C, int dtype, void* stream);
int kad_se_rescale(const void* x, const float* att, void* y, int B, int H, int W, int C, int dtype, void* stream);

/* Tail of KADConv.forward (kad_conv.py:117-121): out = cat_i( upsample_i( y_i * att_i ) ) + x with bilinear
 * upsampling, align_corners = False. Counterpart of k_upsample_bilinear_att / k_cat_residual_att0
 * (kadc_fused_sm75.py:1245-1331).
 *   x, out [B,H,W,C] dtype; y_i [B,H_i,W_i,c_i] dtype, att_i float32 [B][c_i], i = 0..2, sum c_i = C.
 * Optional (set gap[0..2] or none): the channel attention fc (kad_conv.py:104-108,:118) is evaluated inside the
 * kernel from the channel sums the DSC kernels wrote (gap[i] float32 [B][gap_tiles[i]][c_i], mean = sum / (h_i*w_i)),
 * exactly as kad_se_excite does; att[i] must then still point to B*c_i floats, which general shapes use as scratch.
 * out_cstride (0 = C): elements per pixel of `out`, so the result can land in a channel slice of a wider tensor. */
typedef struct KadMergeArgs {
    const void* x; void* out;
    const void* y[3]; const float* att[3];
    int c[3], h[3], w[3];
    int B, H, W, C, dtype;
    const float* gap[3]; const float* fc_w1[3]; const float* fc_b1[3]; const float* fc_w2[3]; const float* fc_b2[3];
    int gap_tiles[3], hidden[3];
    int out_cstride;
} KadMergeArgs;
int kad_merge_upsample_residual(const KadMergeArgs* args, void* stream);

/* A whole KAD-Conv layer in one call: out = KADConv.forward(x) (KAD-Conv/kadconv/kad_conv.py:112-121,
 * == KADC4.forward, KAD-CNet/models/module/KADC/module.py:50-62) for n = 3 branches, BatchNorm folded.
 * The call issues the kernels declared above for the three branches on three streams (the caller's stream and
 * two side streams the library creates once per device on the first call; fork and join by events), so the
 * branches overlap; under stream capture this becomes three parallel chains of the captured graph.
 * Counterpart of the reference's multi-stream branch schedulers (kadc_fused_parallel.py:268-286).
 *   x, out [B,H,W,dim] dtype (NHWC); branch i works at (H >> i) x (W >> i) with c_i channels
 *   (c_0 = dim - 2*(dim/3), c_1 = c_2 = dim/3); parameters float32 as named below;
 *   w_off: kad_dsc_pack_weight_simt of conv_offset.weight; w_dsc_simt: the same of DSC.weight;
 *   w_dsc_tc: kad_dsc_pack_weight_tc of DSC.weight in dtype, or NULL (then, or when the shape does not
 *   qualify, the SIMT kernel runs); ep_scale/ep_shift/ep_post: folded BatchNorm (+ conv bias) and branch scale;
 *   workspace: kad_kadconv_workspace_bytes(B,H,W,dim,dtype,tc_branches) bytes, 256-byte aligned, where bit i of
 *   tc_branches says that branch i passes w_dsc_tc and qualifies for it; status: device int[4] as for kad_dsc_forward.
 * Calls for one device must not be issued concurrently from several host threads (they share the side streams). */
typedef struct KadBranchParams {
    const float* w_proj; const float* b_proj;                       /* [c][dim], [c] */
    const float* lcsa_w1; const float* lcsa_b1; const float* lcsa_bn_scale; const float* lcsa_bn_shift;
    const float* lcsa_w2; const float* lcsa_b2; const float* lcsa_w3; const float* lcsa_b3;
    const float* w_off; const float* b_off;                         /* [9][c][18], [18] */
    const float* w_dsc_simt; const void* w_dsc_tc;
    const void* w_dsc_mma;                                          /* kad_dsc_mma_pack_frags of w_dsc_simt + w_off in dtype, or NULL */
    const float* ep_scale; const float* ep_shift; const float* ep_post;
    const float* fc_w1; const float* fc_b1; const float* fc_w2; const float* fc_b2;   /* [hidden][c], [hidden], [c][hidden], [c] */
    int c, hidden;
} KadBranchParams;
typedef struct KadLayerArgs {
    const void* x; void* out; void* workspace; size_t workspace_bytes; int* status;
    int B, H, W, dim, dtype;
    KadBranchParams br[3];
    int out_cstride;     /* elements per pixel of `out` (0 = dim): the layer can write into a channel slice of a wider tensor */
    int* counters;       /* NULL, or device int[B], zero before the first call and left zero by every call: lets the pyramid kernel
                            finish the LCSA's first stage in its tail (kad_pyramid_project_lcsa) when the shape qualifies */
    int scheme;          /* how the LCSA masks are produced (launches per layer include three squeeze-excite launches and the merge):
                            0 = the library's choice (the fastest measured form: 1);
                            1 = a preparation and a mask kernel per branch, on the branch streams (14 launches per layer);
                            2 = first stage in the pyramid kernel's tail, one mask kernel per branch (11; needs `counters`);
                            3 = first stage in the tail, masks evaluated inside the deformable convolutions (8; needs `counters`);
                            4 = one launch for the three branches' LCSAs, first stage recomputed per block (9).
                            All forms compute bit-identical results. */
} KadLayerArgs;
size_t kad_kadconv_workspace_bytes(int B, int H, int W, int dim, int dtype, int tc_branches);
/* Launches kad_kadconv_forward issues for this shape under `scheme` (as in KadLayerArgs; 0 with_counters = scheme 1). */
int kad_kadconv_launch_count(int B, int H, int W, int dim, int dtype, int tc_branches, int with_counters, int scheme);
int kad_kadconv_forward(const KadLayerArgs* args, void* stream);

/* Batched detection post-processing, one launch for the whole batch. Replaces non_max_suppression
 * (KAD-CNet/utils/general.py:881-990: confidence filter, xywh->xyxy, best class, sort by confidence, class-shifted
 * torchvision.ops.nms at :972, max_det cap) for multi_label = False, agnostic = False.
 *   pred   [B][4+nc][A] dtype: rows 0-3 = cx, cy, w, h in pixels, rows 4.. = class scores (DDetect's y)
 *   dets   float32 [B][max_det][6]: x1, y1, x2, y2, confidence, class, in decreasing confidence; counts int32 [B]
 *   A <= kad_nms_max_anchors() (the sort runs in shared memory), max_det <= 1024; max_wh is the per-class shift (7680).
 * Equal scores keep the lower anchor index first, so the result is deterministic. */
int kad_nms_max_anchors(void);
int kad_nms_batched(const void* pred, int B, int nc, int A, float conf_thres, float iou_thres, int max_det,
                    float max_wh, float* dets, int* counts, int dtype, void* stream);

/* Head decode of one detection scale: distribution-focal-loss expectation, distances to box, sigmoid class scores.
 * Replaces the inference branch of DDetect.forward (KAD-CNet/models/yolo.py:112-127) with DFL (models/common.py:232-243)
 * and make_anchors / dist2bbox (utils/tal/anchor_generator.py:8-32); the reference's own fused version is
 * kadc_head_decode.py:30-88.
 *   raw NHWC [B][H][W][4*reg_max + nc] dtype (box logits side-major: channel = side*reg_max + bin; then class logits),
 *   pred [B][4 + nc][A] dtype: this call writes anchors [a_offset, a_offset + H*W) in (y, x) order: centre x, centre y,
 *   width, height in pixels (cell centre at +0.5, times `stride`), then nc sigmoid scores. fp32 arithmetic. */
int kad_head_decode(const void* raw, void* pred, int B, int H, int W, int reg_max, int nc, float stride,
                    int a_offset, int A, int dtype, void* stream);

/* 1x1 convolution as a tcgen05 GEMM with bias and activation, TMA-fed operands:
 *   y[m, n] = act( sum_k x[m, k] * w[n, k] + bias[n] ),  m over B*H*W pixels.
 * Replaces Conv.forward_fuse for k = 1 (KAD-CNet/models/common.py:56-57 after fuse_conv_and_bn,
 * utils/torch_utils.py:244-265); native counterpart gemm_bias_silu_kernel (kadc_gemm_silu.cu:125-176).
 *   x [M][ldx] dtype (K valid channels, ldx >= K, ldx % 8 == 0), w dtype [N][Kp] with Kp = K rounded up to 8,
 *   bias float32 [N] or NULL, y [M][ldy] dtype. Requires dtype f16/bf16, K % 8 == 0, N % 8 == 0. */
int kad_gemm1x1_tc_supported(int K, int N, int dtype);
int kad_gemm1x1_bias_act(const void* x, const void* w, const float* bias, void* y,
                         long long M, int K, int N, int ldx, int ldy, int act, int dtype,
                         int* status, void* stream);

/* 3x3 convolution (padding 1, stride 1 or 2, dilation 1, one group) as a tcgen05 implicit GEMM with bias and activation:
 *   y[b, yo, xo, n] = act( sum_{ky,kx,c} x[b, s*yo+ky-1, s*xo+kx-1, c] * w[n, ky*3+kx, c] + bias[n] ).
 * Replaces Conv.forward_fuse for k = 3 (KAD-CNet/models/common.py:56-57 after fuse_conv_and_bn,
 * utils/torch_utils.py:244-265), AConv's convolution (common.py:60-67) and the 3x3 convolutions of DDetect
 * (models/yolo.py:95-100); the reference runs them through cuDNN.
 *   x NHWC [B][H][W][ldx] dtype (Cin valid channels from the pointer on, ldx >= Cin, ldx % 8 == 0),
 *   w dtype [Cout][9][Cin] (tap = ky*3+kx), bias float32 [Cout] or NULL,
 *   y NHWC [B][Ho][Wo][ldy] dtype with Ho = (H-1)/s+1, Wo = (W-1)/s+1 (Cout channels written from the pointer on).
 * Requires dtype f16/bf16, Cin % 8 == 0, Cout % 8 == 0. status: 4 ints, zero on entry, non-zero if a wait gave up. */
int kad_conv3x3_tc_supported(int Cin, int Cout, int stride, int dtype);
int kad_conv3x3_bias_act(const void* x, const void* w, const float* bias, void* y,
                         int B, int H, int W, int Cin, int Cout, int stride, int ldx, int ldy, int act, int dtype,
                         int* status, void* stream);

/* The pooling chain of SPPELAN.forward (KAD-CNet/models/common.py:590-598 with SP, :187-193): three chained 5x5 max-pools
 * (stride 1, padding 2) and the torch.cat of the four tensors, in one kernel and in place:
 *   cat NHWC [B][H][W][4*C] dtype; channels [0, C) hold y1 (written there by the 1x1 convolution cv1); the call fills
 *   [C, 2C) = maxpool(y1), [2C, 3C) = maxpool of that, [3C, 4C) = maxpool of that. The reference's own fused version:
 *   sppelin_split_projection (KAD-CNet/inference/acceleration/kadc_fused_nsmall.py:421-443).
 * kad_spp_pool3_supported: dtype f16/bf16, C % 8 == 0 and H*W*32 bytes of shared memory (two planes of 16-byte vectors). */
int kad_spp_pool3_supported(int H, int W, int C, int dtype);
int kad_spp_pool3(void* cat, int B, int H, int W, int C, int dtype, void* stream);

/* Preprocessing of the inference script on the device: letterbox() of KAD-CNet/utils/augmentations.py:106-136 (cv2.resize with
 * INTER_LINEAR to the unpadded size, then a constant border) followed by the BGR->RGB flip and the HWC->CHW transpose of
 * KAD-CNet/inference/infer_dior.py:39-46, for one 8-bit image; the `/255` happens in the detector's first layer
 * (kad_stem_conv_u8). The result equals the OpenCV path bit for bit: same 11-bit fixed-point coefficients and integer passes.
 *   src  uint8 [H0][W0][3] BGR (what cv2.imread returns), dst uint8 [3][Hn][Wn] RGB planes;
 *   the image is resized to new_h x new_w and placed at (top, left); everything else is pad_value (114 in the reference);
 *   xofs int32 [new_w] / xalpha int16 [new_w][2], yofs int32 [new_h] / ybeta int16 [new_h][2]: OpenCV's per-column and per-row
 *   source offsets and coefficients (kadcnet.preprocess.resize_tables computes them on the host as cv::resize does);
 *   area2x = 1 for a shrink by exactly 2 in both directions, which OpenCV computes as the rounded mean of 2x2 blocks (tables unused). */
int kad_letterbox_u8(const void* src_bgr_hwc, void* dst_rgb_chw, int H0, int W0, int Hn, int Wn,
                     int new_h, int new_w, int top, int left, int area2x,
                     const int* xofs, const short* xalpha, const int* yofs, const short* ybeta,
                     int pad_value, void* stream);
/* scale_boxes + clip_boxes + round of the inference script (KAD-CNet/utils/general.py:824-868, infer_dior.py:56) on the padded
 * output of kad_nms_batched: x = clamp((x - pad_x) / gain, 0, width0), y likewise, then round-half-even when do_round.
 *   dets float32 [B][max_det][6] (columns 0-3 are modified in place for the first counts[b] rows of image b), counts int32 [B],
 *   geom float32 [B][5] = gain, pad_x, pad_y, width0, height0 of each image. */
int kad_scale_boxes(float* dets, const int* counts, const float* geom, int B, int max_det, int do_round, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KADCONV_B200_H_ */
