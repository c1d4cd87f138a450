// C-ABI plumbing: error strings, version, and the dispatch of kad_dsc_forward between the SIMT
// kernels, the tcgen05 implicit GEMM and the warp-MMA kernel for small channel counts.
#include <stdarg.h>

#include "kad_common.cuh"

namespace kad {

std::string& last_error() {
    static thread_local std::string s;
    return s;
}

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

int dsc_simt_tiles(int H, int W, int Cin, int Cout);
int launch_dsc_simt(const KadDscArgs& a, cudaStream_t st);
int dsc_tc_tiles(int H, int W);
int launch_dsc_tc(const KadDscArgs& a, cudaStream_t st);
int dsc_mma_tiles(int H, int W);
bool dsc_mma_supported(int Cin, int Cout, int dtype, int H, int W);
bool dsc_mma_inline_mask_supported(int Cin, int Cout, int dtype, int H, int W);
int launch_dsc_mma(const KadDscArgs& a, cudaStream_t st);
size_t dsc_mma_frag_bytes(int Cin, int Cout);
int dsc_mma_pack_frags(const float* w_simt, const float* w_off_simt, void* dst, int Cin, int Cout, int dtype, cudaStream_t st);

}  // namespace kad

using namespace kad;

extern "C" int kad_version(void) { return 100; }

extern "C" int kad_struct_size(int which) {
    switch (which) {
        case 0: return (int)sizeof(KadDscArgs);
        case 1: return (int)sizeof(KadPyramidArgs);
        case 2: return (int)sizeof(KadMergeArgs);
        case 3: return (int)sizeof(KadBranchParams);
        case 4: return (int)sizeof(KadLayerArgs);
        default: return -1;
    }
}

extern "C" const char* kad_last_error_string(void) { return last_error().c_str(); }

extern "C" int kad_dsc_gap_tiles(int H, int W, int Cin, int Cout, int path) {
    if (H <= 0 || W <= 0 || Cin <= 0 || Cout <= 0) return 0;
    if (path == 3) return dsc_mma_tiles(H, W);
    return (path == 1 || path == 2) ? dsc_tc_tiles(H, W) : dsc_simt_tiles(H, W, Cin, Cout);
}

extern "C" int kad_dsc_mma_supported(int Cin, int Cout, int dtype, int H, int W) { return dsc_mma_supported(Cin, Cout, dtype, H, W) ? 1 : 0; }
extern "C" int kad_dsc_mma_inline_mask_supported(int Cin, int Cout, int dtype, int H, int W) { return dsc_mma_inline_mask_supported(Cin, Cout, dtype, H, W) ? 1 : 0; }

extern "C" size_t kad_dsc_mma_frag_bytes(int Cin, int Cout, int dtype) {
    if (!(dtype == KAD_F16 || dtype == KAD_BF16) || Cin < 4 || Cin > 64 || Cout < 1 || Cout > 64) return 0;
    return dsc_mma_frag_bytes(Cin, Cout);
}

extern "C" int kad_dsc_mma_pack_frags(const float* weight_simt, const float* offset_weight_simt, void* dst, int Cin, int Cout, int dtype, void* stream) {
    KAD_CHECK_ARG(weight_simt && offset_weight_simt && dst, "kad_dsc_mma_pack_frags: null pointer");
    KAD_CHECK_ARG(kad_dsc_mma_frag_bytes(Cin, Cout, dtype) != 0, "kad_dsc_mma_pack_frags: needs f16/bf16, 4 <= Cin <= 64, Cout <= 64 (Cin=%d Cout=%d dtype=%d)", Cin, Cout, dtype);
    KAD_CHECK_ARG((uintptr_t)dst % 16 == 0, "kad_dsc_mma_pack_frags: dst must be 16-byte aligned");
    return dsc_mma_pack_frags(weight_simt, offset_weight_simt, dst, Cin, Cout, dtype, (cudaStream_t)stream);
}

extern "C" int kad_dsc_forward(const KadDscArgs* a, void* stream) {
    KAD_CHECK_ARG(a != nullptr, "kad_dsc_forward: null args");
    KAD_CHECK_ARG(a->x && a->weight && a->y, "kad_dsc_forward: null tensor pointer");
    KAD_CHECK_ARG(a->B > 0 && a->H > 0 && a->W > 0 && a->Cin > 0 && a->Cout > 0, "kad_dsc_forward: bad shape B=%d H=%d W=%d Cin=%d Cout=%d",
                  a->B, a->H, a->W, a->Cin, a->Cout);
    KAD_CHECK_ARG(a->B <= 65535, "kad_dsc_forward: batch %d too large", a->B);
    KAD_CHECK_ARG((long long)a->H * a->W < (1ll << 30), "kad_dsc_forward: image too large");
    KAD_CHECK_ARG(a->dtype == KAD_F32 || a->dtype == KAD_F16 || a->dtype == KAD_BF16, "kad_dsc_forward: unknown dtype %d", a->dtype);
    KAD_CHECK_ARG(a->act == KAD_ACT_NONE || a->act == KAD_ACT_SILU || a->act == KAD_ACT_RELU, "kad_dsc_forward: unknown activation %d", a->act);
    if (a->path == 0) return launch_dsc_simt(*a, (cudaStream_t)stream);
    if (a->path == 1 || a->path == 2) {
        if (!kad_dsc_tc_supported(a->Cin, a->Cout, a->dtype))
            return fail(KAD_ERR_UNSUPPORTED, "kad_dsc_forward: tensor path needs f16/bf16, Cin %% 32 == 0, Cout %% 16 == 0, Cout <= 256 (got Cin=%d Cout=%d dtype=%d)",
                        a->Cin, a->Cout, a->dtype);
        KAD_CHECK_ARG(a->status != nullptr, "kad_dsc_forward: the tensor path needs a device status word");
        return launch_dsc_tc(*a, (cudaStream_t)stream);
    }
    if (a->path == 3) {
        if (!dsc_mma_supported(a->Cin, a->Cout, a->dtype, a->H, a->W))
            return fail(KAD_ERR_UNSUPPORTED, "kad_dsc_forward: the warp-MMA path needs f16/bf16, 4 <= Cin <= 64, Cout <= 64 and image rows that fit in shared memory "
                        "(got Cin=%d Cout=%d dtype=%d H=%d W=%d)", a->Cin, a->Cout, a->dtype, a->H, a->W);
        return launch_dsc_mma(*a, (cudaStream_t)stream);
    }
    return fail(KAD_ERR_INVALID, "kad_dsc_forward: unknown path %d", a->path);
}
