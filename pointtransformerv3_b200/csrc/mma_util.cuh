// Small PTX wrappers shared by the warp-level tensor-core kernels.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace ptv3 {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* gptr)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(saddr), "l"(gptr));
}
// 16-byte copy that writes zeros when `valid` is false (nothing is read then)
__device__ __forceinline__ void cp_async16_zfill(uint32_t saddr, const void* gptr, bool valid)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(saddr), "l"(gptr), "r"(valid ? 16 : 0));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t saddr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}

// D += A(16x16, row) * B(16x8, col), bf16 operands, fp32 accumulate
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// two base-2 exponentials of a packed bf16 pair in one instruction
__device__ __forceinline__ uint32_t exp2_bf16x2(uint32_t x)
{
    uint32_t y;
    asm("ex2.approx.ftz.bf16x2 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

// Packed fp32 pairs (two floats in one 64-bit register, one instruction for both).
__device__ __forceinline__ uint64_t pack2(float x, float y)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t r, float& x, float& y)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(r));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// a pair from two 32-bit words (low word = first of the pair)
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
// a bf16x2 word as a pair of floats
__device__ __forceinline__ uint64_t unpack_bf16x2(uint32_t w) { return pack2u(w << 16, w & 0xffff0000u); }
// both floats rounded to bf16 (round to nearest even); `packed` receives the bf16x2 word
__device__ __forceinline__ uint64_t round2(uint64_t v, uint32_t& packed)
{
    float lo, hi;
    unpack2(v, lo, hi);
    packed = pack_bf16(lo, hi);
    return unpack_bf16x2(packed);
}
__device__ __forceinline__ float hsum2(uint64_t v)
{
    float lo, hi;
    unpack2(v, lo, hi);
    return lo + hi;
}

// Constants of the exponentials, packed once per thread.
struct Exp2Const {
    uint64_t log2e, magic, neg_magic, neg_one, c3, c2, c1, one;
    __device__ __forceinline__ Exp2Const()
    {
        log2e = pack2(1.4426950408889634f, 1.4426950408889634f);
        magic = pack2(12582912.f, 12582912.f);
        neg_magic = pack2(-12582912.f, -12582912.f);
        neg_one = pack2(-1.f, -1.f);
        c3 = pack2(0.0555041086f, 0.0555041086f);
        c2 = pack2(0.2402265070f, 0.2402265070f);
        c1 = pack2(0.6931471806f, 0.6931471806f);
        one = pack2(1.f, 1.f);
    }
};

// 2^x for a pair on the FMA pipe: x = n + r with n integer (round to nearest, read off the low
// mantissa bits after adding 1.5 * 2^23) and r in [-0.5, 0.5], 2^r by a cubic (relative error
// 1e-4, far below the bf16 rounding that follows), n added to the exponent field.
__device__ __forceinline__ uint32_t exp2_poly2_bf16(uint64_t x2, const Exp2Const& k)
{
    float x, y;
    unpack2(x2, x, y);
    x2 = pack2(fmaxf(x, -125.f), fmaxf(y, -125.f));
    const uint64_t t2 = add2(x2, k.magic);
    const uint64_t n2 = add2(t2, k.neg_magic);
    const uint64_t r2 = fma2(n2, k.neg_one, x2);
    uint64_t p2 = fma2(r2, k.c3, k.c2);
    p2 = fma2(p2, r2, k.c1);
    p2 = fma2(p2, r2, k.one);
    float px, py, tx, ty;
    unpack2(p2, px, py);
    unpack2(t2, tx, ty);
    px = __int_as_float(__float_as_int(px) + (__float_as_int(tx) << 23));
    py = __int_as_float(__float_as_int(py) + (__float_as_int(ty) << 23));
    return pack_bf16(px, py);
}

}  // namespace ptv3
