// Thin inline-PTX wrappers used by the sm_100a kernels: mbarrier, bulk async
// copies (TMA unit), cp.async, ldmatrix, warp-level MMA, programmatic dependent
// launch, and the nibble / int8 -> half2 converters.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels.h"

namespace nnb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait: gives up after about a tenth of a second of SM clocks and returns false
// (the caller records an error status and carries on; nothing spins forever).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit_cycles = 200000000ll) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit_cycles) return false;
    }
}

// Warp-wide form for long waits (a whole K loop): one lane polls, with a suspend-time hint so that
// the hardware parks it between polls, and the result is shared by shuffle.  Thirty-two lanes
// spinning on the same barrier would only take issue slots from the warps that do the work.
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint32_t bar, uint32_t parity, long long limit_cycles = 200000000ll) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) {
        const long long t0 = clock64();
        for (;;) {
            uint32_t done;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(bar), "r"(parity), "r"(4000u)
                : "memory");
            if (done) break;
            if (clock64() - t0 > limit_cycles) {
                ok = 0;
                break;
            }
        }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

// ---- bulk async copy global -> shared (1-D, TMA unit) --------------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

// ---- tiled 2-D tensor copy global -> shared (TMA unit, 128-byte swizzle set in the map) ----
// x = coordinate in the innermost dimension (elements; must cover a multiple of 16 bytes),
// y = row.  The whole box is written (out-of-range parts as zeros) and counted on the mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- cp.async (per-thread, 4/16-byte) tracked by an mbarrier -------------------
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- ldmatrix / mma ------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B + C with C in registers of its own (the accumulator starts from a given value)
__device__ __forceinline__ void mma_16816_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                            const float4& c) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}

// D(16x8,s32) += A(16x32,s8,row) * B(32x8,col); B is signed or unsigned 8-bit
template <bool B_SIGNED>
__device__ __forceinline__ void imma_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if (B_SIGNED)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- programmatic dependent launch ----------------------------------------------
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- exact integer -> half2 converters -------------------------------------------
// 4 int8 in one word -> two half2 holding (q0,q1) and (q2,q3), exact.
// Bias the bytes to unsigned, drop each into the mantissa of 1024.0h, subtract 1152.
__device__ __forceinline__ void int8x4_to_half2x2(uint32_t w, uint32_t& h01, uint32_t& h23) {
    const uint32_t u = w ^ 0x80808080u;
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(u), "r"(0x64646464u));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(u), "r"(0x64646464u));
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1152
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
    __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
    h01 = *reinterpret_cast<uint32_t*>(&ha);
    h23 = *reinterpret_cast<uint32_t*>(&hb);
}

// 8 nibbles in one word -> four half2 of (nibble - 8), exact, paired as
// (n0,n4) (n1,n5) (n2,n6) (n3,n7)  [n_i = bits 4i..4i+3].
__device__ __forceinline__ void q4x8_to_half2x4(uint32_t w, uint32_t& p04, uint32_t& p15, uint32_t& p26, uint32_t& p37) {
    const uint32_t MAGIC = 0x64006400u;  // 1024.0h in both lanes
    uint32_t lo0, hi0, lo1, hi1;
    const uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(lo0) : "r"(w), "r"(0x000F000Fu), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(hi0) : "r"(w), "r"(0x00F000F0u), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(lo1) : "r"(w8), "r"(0x000F000Fu), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(hi1) : "r"(w8), "r"(0x00F000F0u), "r"(MAGIC));
    const __half2 b1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));  // 1024 + 8
    const __half2 sixteenth = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));  // 1/16
    const __half2 m72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));        // -(64 + 8)
    __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&lo0), b1032);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2*>(&hi0), sixteenth, m72);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2*>(&lo1), b1032);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&hi1), sixteenth, m72);
    p04 = *reinterpret_cast<uint32_t*>(&r0);
    p15 = *reinterpret_cast<uint32_t*>(&r1);
    p26 = *reinterpret_cast<uint32_t*>(&r2);
    p37 = *reinterpret_cast<uint32_t*>(&r3);
}

// 8 nibbles in one word -> four half2 of (64 + nibble), exact, paired as
// (n0,n4) (n1,n5) (n2,n6) (n3,n7): each nibble is moved to mantissa bits 4..7 of 64.0h.
// The common offset 64 + 8 is taken out of the 32-weight block sum afterwards
// (sum (64 + n) x - 72 sum x = sum (n - 8) x), so no subtraction is spent per weight.
constexpr float Q4_BIAS = 72.0f;
__device__ __forceinline__ void q4x8_to_half2x4_biased(uint32_t w, uint32_t& p04, uint32_t& p15, uint32_t& p26, uint32_t& p37) {
    const uint32_t MASK = 0x00F000F0u, MAGIC = 0x54005400u;  // 64.0h in both lanes
    const uint32_t wl4 = w << 4, wr4 = w >> 4, wr8 = w >> 8;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(p04) : "r"(wl4), "r"(MASK), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(p15) : "r"(w), "r"(MASK), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(p26) : "r"(wr4), "r"(MASK), "r"(MAGIC));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(p37) : "r"(wr8), "r"(MASK), "r"(MAGIC));
}

// Order-preserving arg-max key of an fp16 value: larger value wins, then the LOWER index.
__device__ __forceinline__ unsigned long long argmax_key_half(uint16_t h, int idx) {
    unsigned int b = __float_as_uint(__half2float(__ushort_as_half(h)));
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}

// Called by one thread of every block after a barrier that covers the block's output stores
// (kernels.h: GatherSignal).  Every block orders its stores, local and to peers, before its
// count with a device-scope fence; the block that completes the count publishes the epoch with
// one system-scope release, which is cumulative over what the counts it observed had ordered.
// System-scope fences cost microseconds each, so there is exactly one on this path.
// Row-sharded greedy pick: this rank's best key (ordered fp32 bits of an fp16 value << 32 |
// ~global row; 0 = no candidate) goes, re-packed as pick number (16 bits) | ordered fp16 value
// (16) | ~row (32), into word `rank` of every rank's key table, which follows the flag words in
// the same symmetric allocation.  The word carries its own arrival mark, so no fence or flag
// accompanies it.  Two tables alternate with the pick number: a rank already one pick ahead
// cannot overwrite a word that a slower rank has not read yet, and it cannot be two ahead because
// its own next pick waits for every rank's word.  `s.epoch` counts this rank's picks here.
// Called by one thread of the block that finishes the launch's arg-max.
__device__ __forceinline__ void argmax_share_key(const nnb::GatherSignal& s, unsigned long long key) {
    const unsigned e = *reinterpret_cast<volatile unsigned*>(s.epoch) + 1u;
    *reinterpret_cast<volatile unsigned*>(s.epoch) = e;
    unsigned long long payload = 0ull;
    if (key) {
        const unsigned ob = (unsigned)(key >> 32);
        const unsigned fb = (ob & 0x80000000u) ? (ob & 0x7FFFFFFFu) : ~ob;  // back to the float's bits
        const unsigned h = __half_as_ushort(__float2half_rn(__uint_as_float(fb)));  // exact: the value is an fp16
        const unsigned oh = (h & 0x8000u) ? (~h & 0xFFFFu) : (h | 0x8000u);       // never 0 for a non-NaN
        payload = ((unsigned long long)oh << 32) | (key & 0xFFFFFFFFull);
    }
    const unsigned long long word = ((unsigned long long)(e & 0xFFFFu) << 48) | payload;
    for (int g = 0; g < s.world; ++g) {
        unsigned long long* dst =
            reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(s.flags[g]) + nnb::KEY_TABLE_OFFSET) + (e & 1u) * 8u + (unsigned)s.rank;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
    }
}

// Two invariants this signalling rests on:
//  (1) Ordering of the peer stores.  Every block orders its own stores (local and peer) before its count-in with a
//      gpu-scope fence; the last block to count in observes all the others through the atomic and issues the one
//      system-scope fence before it writes the flags, so the other blocks' peer stores become visible to the peers by
//      cumulativity (valid under the PTX memory model; the stress loop of tests/multi_gpu_worker.py compares several
//      hundred gathers bit for bit with NCCL's).
//  (2) Nothing after this call in the projection kernel may touch state that the next launch on the stream reads: the
//      wait and pick kernels are launched programmatically and never execute griddepcontrol.wait (their own rank's flag
//      is among those they spin on), so the launch after them is not ordered behind the projection grid's retirement,
//      only behind its signal.
__device__ __forceinline__ void gather_signal_block_done(const nnb::GatherSignal& s) {
    __threadfence();
    const unsigned prev = atomicAdd(s.done, 1u);
    if (prev == gridDim.x - 1u) {
        *reinterpret_cast<volatile unsigned*>(s.done) = 0u;
        const unsigned e = *reinterpret_cast<volatile unsigned*>(s.epoch) + 1u;
        *reinterpret_cast<volatile unsigned*>(s.epoch) = e;
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        for (int g = 0; g < s.world; ++g) {
            unsigned* dst = s.flags[g] + s.rank;
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(e) : "memory");
        }
    }
}

}  // namespace nnb
