// Helpers shared by the warp-level tensor-core kernels (mma.sync m16n8k16, fp16/bf16 operands, fp32 accumulators):
// packed conversions, the MMA itself, 8-byte operand loads with a known alignment, cp.async.
#pragma once
#include "kad_common.cuh"

namespace kad {
namespace {

constexpr int MMA_THREADS = 256;

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ uint32_t mul2(uint32_t x, uint32_t w);
template <> __device__ __forceinline__ uint32_t mul2<__half>(uint32_t x, uint32_t w) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&x), *reinterpret_cast<__half2*>(&w)); return *reinterpret_cast<uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t mul2<__nv_bfloat16>(uint32_t x, uint32_t w) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&x), *reinterpret_cast<__nv_bfloat162*>(&w)); return *reinterpret_cast<uint32_t*>(&r);
}

template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b);
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint2 b) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b.x), "r"(b.y));
}


// Eight bytes (four consecutive 16-bit channels) at byte offset `off` of the block's shared memory, whose address is
// known to be ALIGN-byte aligned. ALIGN = 2 reads the three aligned words around the span and shifts the bytes outside
// it away (the staged window has slack on both sides for exactly this).
template <int ALIGN>
__device__ __forceinline__ uint2 lds8(const unsigned char* smem, uint32_t off) {
    if (ALIGN >= 8) return *reinterpret_cast<const uint2*>(smem + off);
    if (ALIGN == 4) { const uint32_t* q = reinterpret_cast<const uint32_t*>(smem + off); return make_uint2(q[0], q[1]); }
    const uint32_t* q = reinterpret_cast<const uint32_t*>(smem + (off & ~3u));
    const uint32_t sh = (off & 2u) * 8u;
    return make_uint2(__funnelshift_r(q[0], q[1], sh), __funnelshift_r(q[1], q[2], sh));
}
// The same through a global pointer; here the word after the span is only read when the span ends inside it.
template <int ALIGN>
__device__ __forceinline__ uint2 ldg8(const unsigned char* p) {
    if (ALIGN >= 8) return __ldg(reinterpret_cast<const uint2*>(p));
    if (ALIGN == 4) { const uint32_t* q = reinterpret_cast<const uint32_t*>(p); return make_uint2(__ldg(q), __ldg(q + 1)); }
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
    const bool odd = (a & 2) != 0;
    const uint32_t w0 = __ldg(q), w1 = __ldg(q + 1), w2 = odd ? __ldg(q + 2) : 0u;
    return odd ? make_uint2(__funnelshift_r(w0, w1, 16), __funnelshift_r(w1, w2, 16)) : make_uint2(w0, w1);
}

// Which four channels lane t gathers in 16-channel chunk kc: normally ch = kc*16 + 4t .. ch+3. In the last, partial
// chunk a lane with only 1-3 existing channels loads the LAST four channels of the pixel instead, and a lane with none
// re-reads channels 0-3; the weight fragments (stage_weights) carry zeros for every slot that would count a channel
// twice, so no lane ever reads past its pixel and no masking is needed in the gather.
__device__ __forceinline__ int lane_first_channel(int kc, int t, int Cin) {
    const int ch = kc * 16 + 4 * t, nv = Cin - ch;
    return nv >= 4 ? ch : (nv <= 0 ? 0 : Cin - 4);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most one committed group is still in flight
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

}  // namespace
}  // namespace kad
