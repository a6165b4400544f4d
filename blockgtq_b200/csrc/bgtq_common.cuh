// Device-side helpers shared by the sm_100a kernels: PTX wrappers for bulk
// (TMA) copies with mbarrier completion, bounded mbarrier waits, warp-level
// tensor-core MMA and small bit utilities.
//
// The decode kernel is also compiled at run time (NVRTC) from this very text, with BGTQ_JIT defined and
// no headers available: everything it needs is written with built-ins and inline PTX, and the parts that
// need CUDA's headers are fenced off.
#pragma once

#ifndef BGTQ_JIT
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bgtq.h"
#endif

namespace bgtq {

constexpr int kHD = BGTQ_HEAD_DIM;

// Error codes a kernel may leave in the caller's status word.
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusOverflow = 2;     // an append at a device-side position would leave the cache

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Wait with an iteration limit: returns false if the phase never completed.
// try_wait itself blocks for a hardware-defined slice, so the bound below is
// on the order of a second of wall time, far beyond any legitimate wait.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// ---- bulk async copy global -> shared (1-D TMA) -----------------------------
// dst and src 16-byte aligned, bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Same copy with an L2 evict-first policy: for data that is read once per launch (the packed cache
// stream), so it does not push the small hot tables of other kernels out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// ---- shared memory loads -----------------------------------------------------
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// 32 bits starting at an arbitrary BIT position of a byte stream in shared
// memory (two aligned words + funnel shift).  Reads up to 7 bytes past the
// last needed byte: buffers carry that much slack.
__device__ __forceinline__ uint32_t lds_bits32(uint32_t base_addr, uint32_t bitpos) {
    const uint32_t a = base_addr + (bitpos >> 3);
    const uint32_t wa = a & ~3u;
    const uint32_t sh = ((a & 3u) << 3) + (bitpos & 7u);
    return __funnelshift_r(lds32(wa), lds32(wa + 4), sh);
}
// 64 bits starting at an arbitrary bit position (three aligned words).
__device__ __forceinline__ uint2 lds_bits64(uint32_t base_addr, uint32_t bitpos) {
    const uint32_t a = base_addr + (bitpos >> 3);
    const uint32_t wa = a & ~3u;
    const uint32_t sh = ((a & 3u) << 3) + (bitpos & 7u);
    const uint32_t w0 = lds32(wa), w1 = lds32(wa + 4), w2 = lds32(wa + 8);
    return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
}

// ---- tensor core -------------------------------------------------------------
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// D(16x8,f32) = A * B  (zero accumulator input)
__device__ __forceinline__ void mma_16816_z(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(0.f));
}
// Transpose an 8x8 tile of 16-bit values held one row-pair per thread.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// fp16 arithmetic on raw bit patterns (round to nearest even, no flush): what __floats2half2_rn, __hmul2
// and __half2float compile to.
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float f16_bits_to_float(uint32_t h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((unsigned short)h));
    return f;
}

// Programmatic dependent launch (a kernel launched with the stream-serialization attribute may start
// while its predecessor in the stream still runs).  grid_launch_dependents lets the NEXT kernel's blocks
// become resident early; grid_dependency_wait blocks until the PREVIOUS kernel has completed and its
// writes are visible.  Both are no-ops for a kernel launched the ordinary way.  Every kernel of a chain
// executes the wait before it ends, so completion stays transitive along the stream.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifndef BGTQ_JIT
// Launch with or without the programmatic stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool programmatic, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    return e == cudaSuccess ? cudaGetLastError() : e;
}
#endif

__host__ __device__ __forceinline__ int seg_storage_bytes(int bw, int n) {
    return bw == 1 ? (n + 7) / 8 : bw == 2 ? (n + 3) / 4 : bw == 3 ? ((n + 7) / 8) * 3 : bw == 4 ? (n + 1) / 2 : n;
}

}  // namespace bgtq
