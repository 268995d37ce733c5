// Minimal OpenCL C -> C++ shim (TEST INFRASTRUCTURE ONLY).
//
// Lets the reference's unmodified .cl kernel sources for the decode GEMV path be
// compiled by g++ and run on the host, so that the CPU oracle can be pinned against
// the reference's own kernel code.  oracle/build_ref.py prepends this header to each
// .cl file (read from the reference checkout where it lies; nothing is copied into
// this repository) and appends a generated name -> call dispatcher.
//
// What is emulated: address-space qualifiers, half / float4 / int4 / uint4,
// vload_half / vload_half4 / vstore_half (round to nearest even), image2d_t reads
// of RGBA int8 / uint8 / half pixels over a row-major weight matrix, dot,
// convert_float4, native_exp, work-item ids, and barrier() (the 64 work-items of a
// group run as cooperative fibers; barrier() yields to the next fiber).
// dot() is evaluated left to right with separate multiplies and adds; the file is
// built with -ffp-contract=off, so results do not depend on FMA contraction.
#pragma once
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <ucontext.h>

#include <functional>
#include <vector>

// ---- qualifiers ----------------------------------------------------------------
#define __kernel static
#define __global
#define __constant
#define __read_only
#define __write_only
#define __local static thread_local
#define CLK_LOCAL_MEM_FENCE 1
#define CLK_GLOBAL_MEM_FENCE 2
#define CLK_NORMALIZED_COORDS_FALSE 0
#define CLK_ADDRESS_NONE 0
#define CLK_ADDRESS_CLAMP 0
#define CLK_FILTER_NEAREST 0
#ifndef FLT_MAX
#define FLT_MAX 3.402823466e+38f
#endif

typedef unsigned int uint;
typedef unsigned char uchar;
typedef int sampler_t;

// ---- half ------------------------------------------------------------------------
static inline float clshim_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (!man) bits = sign;
        else {
            int sh = 0;
            while (!(man & 0x400u)) { man <<= 1; ++sh; }
            bits = sign | ((uint32_t)(113 - sh) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
static inline uint16_t clshim_f2h(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    uint32_t e8 = (b >> 23) & 0xFFu, man = b & 0x7FFFFFu;
    if (e8 == 0xFFu) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0u));
    int32_t e = (int32_t)e8 - 112;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e), q = man >> shift, rem = man & ((1u << shift) - 1u), hf = 1u << (shift - 1);
        if (rem > hf || (rem == hf && (q & 1u))) ++q;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)e << 10) | (man >> 13), rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) ++q;
    return (uint16_t)(sign | q);
}

struct half {
    uint16_t bits;
    operator float() const { return clshim_h2f(bits); }
};

// ---- vectors -----------------------------------------------------------------------
struct float4 {
    union { struct { float x, y, z, w; }; struct { float s0, s1, s2, s3; }; };
    float4() = default;
    float4(float v) : x(v), y(v), z(v), w(v) {}  // the literal form (float4)(v) splats
};
struct int4 { int x, y, z, w; };
struct uint4 { uint x, y, z, w; };
struct cl_int2_t { int x, y; };
static inline cl_int2_t cl_make_int2(int a, int b) { return cl_int2_t{a, b}; }
#define int2 cl_make_int2  // the kernels only use the literal form (int2)(a, b)

static inline float4 mk4(float a, float b, float c, float d) { float4 r; r.x = a; r.y = b; r.z = c; r.w = d; return r; }
static inline float4 operator+(float4 a, float4 b) { return mk4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
static inline float4 operator*(float4 a, float4 b) { return mk4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
static inline float4& operator+=(float4& a, float4 b) { a = a + b; return a; }
static inline float4 convert_float4(int4 v) { return mk4((float)v.x, (float)v.y, (float)v.z, (float)v.w); }
static inline float4 convert_float4(uint4 v) { return mk4((float)v.x, (float)v.y, (float)v.z, (float)v.w); }
static inline float4 convert_float4(float4 v) { return v; }
static inline float dot(float4 a, float4 b) { return ((a.x * b.x + a.y * b.y) + a.z * b.z) + a.w * b.w; }
static inline float native_exp(float x) { return expf(x); }
static inline float native_recip(float x) { return 1.0f / x; }
static inline float native_rsqrt(float x) { return 1.0f / sqrtf(x); }
static inline int min(int a, int b) { return a < b ? a : b; }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline int atomic_add(int* p, int v) { int o = *p; *p += v; return o; }

static inline float vload_half(size_t off, const half* p) { return clshim_h2f(p[off].bits); }
static inline float4 vload_half4(size_t off, const half* p) {
    const half* q = p + 4 * off;
    return mk4(clshim_h2f(q[0].bits), clshim_h2f(q[1].bits), clshim_h2f(q[2].bits), clshim_h2f(q[3].bits));
}
static inline void vstore_half(float v, size_t off, half* p) { p[off].bits = clshim_f2h(v); }
static inline void vstore_half4(float4 v, size_t off, half* p) {
    half* q = p + 4 * off;
    q[0].bits = clshim_f2h(v.x); q[1].bits = clshim_f2h(v.y); q[2].bits = clshim_f2h(v.z); q[3].bits = clshim_f2h(v.w);
}
static inline float vload_half(size_t off, const float* p) { return p[off]; }

// ---- images: a 2-D view over the row-major weight matrix ---------------------------
// One pixel = 4 channels; `pitch` is the byte distance between image rows.
struct image2d_t {
    const uint8_t* data;
    size_t pitch;
};
static inline int4 read_imagei(image2d_t img, sampler_t, cl_int2_t c) {
    const int8_t* p = (const int8_t*)(img.data + (size_t)c.y * img.pitch + (size_t)c.x * 4);
    return int4{p[0], p[1], p[2], p[3]};
}
static inline uint4 read_imageui(image2d_t img, sampler_t, cl_int2_t c) {
    const uint8_t* p = img.data + (size_t)c.y * img.pitch + (size_t)c.x * 4;
    return uint4{p[0], p[1], p[2], p[3]};
}
static inline float4 read_imageh(image2d_t img, sampler_t, cl_int2_t c) {
    const uint16_t* p = (const uint16_t*)(img.data + (size_t)c.y * img.pitch + (size_t)c.x * 8);
    return mk4(clshim_h2f(p[0]), clshim_h2f(p[1]), clshim_h2f(p[2]), clshim_h2f(p[3]));
}
static inline float4 read_imagef(image2d_t img, sampler_t s, cl_int2_t c) { return read_imageh(img, s, c); }

// ---- work-item ids and barrier: one work-group = cooperative fibers on one thread ----
namespace clshim {
struct Fiber {
    ucontext_t ctx;
    std::vector<char> stack;
    bool done = false;
};
struct GroupState {
    size_t group_id = 0, local_size = 1, num_groups = 1;
    size_t local_id = 0;
    ucontext_t sched;
    Fiber* cur = nullptr;
    const std::function<void()>* body = nullptr;
};
static thread_local GroupState g_gs;

static void trampoline() {
    (*g_gs.body)();
    g_gs.cur->done = true;
    swapcontext(&g_gs.cur->ctx, &g_gs.sched);
}

// Run groups [g0, g1) of `local_size` work-items each on the calling thread.
static inline void run_groups(size_t g0, size_t g1, size_t num_groups, size_t local_size, const std::function<void()>& body) {
    std::vector<Fiber> fibers(local_size);
    for (auto& f : fibers) f.stack.resize(64 * 1024);
    g_gs.local_size = local_size;
    g_gs.num_groups = num_groups;
    g_gs.body = &body;
    for (size_t g = g0; g < g1; ++g) {
        g_gs.group_id = g;
        for (size_t t = 0; t < local_size; ++t) {
            Fiber& f = fibers[t];
            f.done = false;
            getcontext(&f.ctx);
            f.ctx.uc_stack.ss_sp = f.stack.data();
            f.ctx.uc_stack.ss_size = f.stack.size();
            f.ctx.uc_link = nullptr;
            makecontext(&f.ctx, (void (*)())trampoline, 0);
        }
        size_t remaining = local_size;
        while (remaining) {
            remaining = 0;
            for (size_t t = 0; t < local_size; ++t) {
                Fiber& f = fibers[t];
                if (f.done) continue;
                g_gs.cur = &f;
                g_gs.local_id = t;
                swapcontext(&g_gs.sched, &f.ctx);
                if (!f.done) ++remaining;
            }
        }
    }
}
}  // namespace clshim

static inline size_t get_group_id(int) { return clshim::g_gs.group_id; }
static inline size_t get_local_id(int) { return clshim::g_gs.local_id; }
static inline size_t get_local_size(int) { return clshim::g_gs.local_size; }
static inline size_t get_num_groups(int) { return clshim::g_gs.num_groups; }
static inline size_t get_global_id(int) { return clshim::g_gs.group_id * clshim::g_gs.local_size + clshim::g_gs.local_id; }
static inline size_t get_global_size(int) { return clshim::g_gs.num_groups * clshim::g_gs.local_size; }
static inline void barrier(int) { swapcontext(&clshim::g_gs.cur->ctx, &clshim::g_gs.sched); }
