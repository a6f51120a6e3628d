// Device code shared by the single-row W4A16 kernels (w4_gemv1.cu: one linear; moe_decode.cu: the picks of a routed
// layer): the offset-free nibble expansion, the staging of one activation row in the order the fragments read it, and
// small helpers.
#pragma once
#include "w4_tile.cuh"

namespace eq {

constexpr int kG1Warps = 16;
constexpr int kG1Threads = kG1Warps * 32;
constexpr int kG1Slot = 1024 + 256;  // ring slot: the item's nibbles, then one private 8-byte scale / zero entry per lane

template <typename ActT>
struct Raw;
template <>
struct Raw<__half> {
    static constexpr float kOffset = 1024.f;
    static constexpr bool kPrescaleHi = true;
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x64006400u;
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w, 0x00F000F0u, kMagic);
        const uint32_t w8 = w >> 8;
        a[1] = lop3<0xEA>(w8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w8, 0x00F000F0u, kMagic);
    }
    static __device__ __forceinline__ uint32_t sixteenth(uint32_t pair) {
        uint32_t r;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(pair), "r"(0x2C002C00u));
        return r;
    }
    static __device__ __forceinline__ float pair_sum(uint32_t pair) {
        const __half2 h = *reinterpret_cast<const __half2*>(&pair);
        return __low2float(h) + __high2float(h);
    }
};
template <>
struct Raw<__nv_bfloat16> {
    static constexpr float kOffset = 128.f;
    static constexpr bool kPrescaleHi = false;
    static __device__ __forceinline__ void expand(uint32_t w, uint32_t (&a)[4]) {
        constexpr uint32_t kMagic = 0x43004300u;
        a[0] = lop3<0xEA>(w, 0x000F000Fu, kMagic);
        a[2] = lop3<0xEA>(w >> 4, 0x000F000Fu, kMagic);
        a[1] = lop3<0xEA>(w >> 8, 0x000F000Fu, kMagic);
        a[3] = lop3<0xEA>(w >> 12, 0x000F000Fu, kMagic);
    }
    static __device__ __forceinline__ uint32_t sixteenth(uint32_t pair) { return pair; }
    static __device__ __forceinline__ float pair_sum(uint32_t pair) {
        return __uint_as_float(pair << 16) + __uint_as_float(pair & 0xFFFF0000u);
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// n / d for 0 <= n < 2^30 by one multiply: inv = floor(2^32 / d) + 1 overestimates the quotient by at most one.
__device__ __forceinline__ int quotient(int n, int d, uint32_t inv) {
    if (inv == 0) return n;  // d == 1
    int q = static_cast<int>(__umulhi(static_cast<uint32_t>(n), inv));
    if (q * d > n) --q;
    return q;
}


// Stages vector v (eight consecutive activations, v = 16 item + 4 j + q) of a row: the high k-slots pre-divided by 16,
// stored as [item][chunk c][lane column j] of 16 bytes (chunk c of lane column j holds the {low slot, high slot} word
// pairs of k16 steps 2c and 2c + 1), and adds up the item's two sums {offset S1, S2}.  Call with whole warps: the sums
// are shuffled over the sixteen lanes of an item; `live` is false for the padding lanes beyond the row.
template <typename ActT>
__device__ __forceinline__ void stage_vector(uint4 val, int v, bool live, uint4* xs, float2* xsum) {
    // rows 16..31 of every 32-row lane block are the high k-slots: vectors 2, 3 of every four
    float s2 = Raw<ActT>::pair_sum(val.x) + Raw<ActT>::pair_sum(val.y) + Raw<ActT>::pair_sum(val.z) + Raw<ActT>::pair_sum(val.w);
    float s1 = s2;
    if (Raw<ActT>::kPrescaleHi && (v & 2)) {
        val.x = Raw<ActT>::sixteenth(val.x);
        val.y = Raw<ActT>::sixteenth(val.y);
        val.z = Raw<ActT>::sixteenth(val.z);
        val.w = Raw<ActT>::sixteenth(val.w);
        s1 = Raw<ActT>::pair_sum(val.x) + Raw<ActT>::pair_sum(val.y) + Raw<ActT>::pair_sum(val.z) + Raw<ActT>::pair_sum(val.w);
    }
    if (live) {
        // q & 1 picks steps 0..3 / 4..7, q >> 1 the low / high slots; word i of the vector is step s = 4 (q & 1) + i:
        // chunk s / 2, word 2 (s & 1) + (q >> 1) of the chunk
        const int q = v & 3, jj = (v >> 2) & 3, item = v >> 4;
        uint32_t* dst = reinterpret_cast<uint32_t*>(xs) + item * 64 + (2 * (q & 1)) * 16 + jj * 4 + (q >> 1);
        dst[0] = val.x;   // step 4 (q & 1)
        dst[2] = val.y;   // step 4 (q & 1) + 1: same chunk, next pair
        dst[16] = val.z;  // next chunk
        dst[18] = val.w;
    }
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) {
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, off);
        s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, off);
    }
    if (live && (v & 15) == 0) xsum[v >> 4] = make_float2(Raw<ActT>::kOffset * s1, s2);
}

// One item: the lane's 2 x 16 weight bytes and its scale / zero entry from the ring slot at `w_addr` / `m_addr`, the
// staged activations at `x_addr` and the item's sums at `sum_addr`; adds s (acc - 1024 S1 - z S2) for columns g and
// g + 8 into y_lo / y_hi (live in lanes with j == 0).
template <typename ActT, bool SCALE_F16>
__device__ __forceinline__ void gemv1_item(uint32_t w_addr, uint32_t m_addr, uint32_t x_addr, uint32_t sum_addr, float& y_lo, float& y_hi) {
    uint32_t w[8], m0, m1, xv[16];
    float sum1, sum2;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(w_addr) : "memory");
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+512];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(w_addr) : "memory");
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(m0), "=r"(m1) : "r"(m_addr) : "memory");
    // the B fragments of the eight k16 steps.  Only column 0 of the 16 x 8 product is ever looked at (its B values sit
    // in lanes 0..3); every lane of a column j reads the same 64 bytes, so all eight columns are copies.
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xv[0]), "=r"(xv[1]), "=r"(xv[2]), "=r"(xv[3]) : "r"(x_addr) : "memory");
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+64];" : "=r"(xv[4]), "=r"(xv[5]), "=r"(xv[6]), "=r"(xv[7]) : "r"(x_addr) : "memory");
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+128];" : "=r"(xv[8]), "=r"(xv[9]), "=r"(xv[10]), "=r"(xv[11]) : "r"(x_addr) : "memory");
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+192];" : "=r"(xv[12]), "=r"(xv[13]), "=r"(xv[14]), "=r"(xv[15]) : "r"(x_addr) : "memory");
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(sum1), "=f"(sum2) : "r"(sum_addr) : "memory");
    constexpr int kChains = 2;  // independent accumulator chains (four were slower: registers)
    float acc[kChains][4];
#pragma unroll
    for (int st = 0; st < 8; ++st) {
        uint32_t a[4];
        Raw<ActT>::expand(w[st], a);
        // staged as {low slot, high slot} word pairs per k16 step
        if (st < kChains)
            Frag<ActT>::mma0(acc[st % kChains], a, xv[2 * st], xv[2 * st + 1]);
        else
            Frag<ActT>::mma(acc[st % kChains], a, xv[2 * st], xv[2 * st + 1]);
    }
    float s_lo, s_hi;
    if (SCALE_F16) {
        const __half2 sc = *reinterpret_cast<const __half2*>(&m0);
        s_lo = __low2float(sc);
        s_hi = __high2float(sc);
    } else {
        s_lo = __uint_as_float(m0 << 16);
        s_hi = __uint_as_float(m0 & 0xFFFF0000u);
    }
    const __half2 z = *reinterpret_cast<const __half2*>(&m1);
    // c0: column g, c2: column g + 8 of row 0 of the product, both in lanes j == 0
    y_lo = fmaf(s_lo, (acc[0][0] + acc[1][0]) - fmaf(__low2float(z), sum2, sum1), y_lo);
    y_hi = fmaf(s_hi, (acc[0][2] + acc[1][2]) - fmaf(__high2float(z), sum2, sum1), y_hi);
}

}  // namespace eq
