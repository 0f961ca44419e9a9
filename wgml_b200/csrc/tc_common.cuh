// Pieces shared by the kernels that use the fifth-generation tensor cores (tcgen05.mma kind::i8 with the
// accumulators in tensor memory): operand and instruction descriptors, the issue / commit / load wrappers and
// the bounded wait of a block that winds down as a whole once one of its waits has expired.
#pragma once

#include "async_copy.cuh"
#include "gemv_core.cuh"

namespace wgb {

constexpr uint32_t TC_TILE_ROWS = 128;
constexpr uint32_t TC_UNIT_BYTES = TC_TILE_ROWS * 144;        // one super-block column of a tile, raw
constexpr uint32_t TC_A_BYTES = TC_TILE_ROWS * 256;           // the same, unpacked to bytes

// 64-bit shared-memory operand descriptor, no swizzle, K-major operand: start address, the byte distance
// between core matrices (8 rows x 16 bytes) adjacent along K ("leading" field) and the distance between
// those adjacent along the rows ("stride" field).  Checked against the dp4a kernel on the device.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((leading_bytes & 0x3ffffu) >> 4) << 16;
    d |= (uint64_t)((stride_bytes & 0x3ffffu) >> 4) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version of this architecture
    return d;
}
// The same for a K-major operand in the 128-byte swizzled layout: rows of 128 bytes, groups of 8 rows
// (1024 bytes, `group_bytes` apart), the 16-byte chunks of row i stored at chunk index ^ (i % 8).  A step
// along K inside the 128 bytes is a plain byte offset on the start address (tile base on a 1 KB boundary).
__device__ __forceinline__ uint64_t tc_smem_desc_sw128(uint32_t addr, uint32_t group_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((group_bytes & 0x3ffffu) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;   // 128-byte swizzle
    return d;
}

// kind::i8 instruction descriptor: D s32, A u8 (or s8 with `a_signed`), B s8, both K-major, M = 128, N = n (a
// multiple of 16).
__device__ __forceinline__ uint32_t tc_idesc(uint32_t n, uint32_t a_signed = 0)
{
    return (2u << 4) | (a_signed << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, 0, 0;\n\t"   // do not accumulate: D = A * B
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
// The same with the accumulate flag as an argument: D = A * B (+ D when `accumulate`).
__device__ __forceinline__ void tc_mma_acc(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, int (&v)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_ld2(uint32_t taddr, int (&v)[2])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld4(uint32_t taddr, int (&v)[4])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
}

// Bounded wait (in time) that also gives up when another thread of the block already has.  A poll may park the
// thread for up to TC_POLL_NS, so the untimed polls below cover at most a few hundred microseconds.
#ifndef TC_POLL_NS
#define TC_POLL_NS 1000u
#endif
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile uint32_t *dead, uint32_t *err, uint32_t code)
{
#pragma unroll 1
    for (int i = 0; i < 256; i++) {
        if (mbar_try_wait_hint(bar, parity, TC_POLL_NS)) return true;
        if ((i & 15) == 15 && *dead) return false;
    }
    const unsigned long long t0 = global_ns();
    do {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait_hint(bar, parity, TC_POLL_NS)) return true;
        if (*dead) return false;
    } while (global_ns() - t0 < ASYNC_WAIT_NS);
    *dead = 1;
    if (err) atomicCAS(err, 0u, code);
    return false;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Units of a block: items blockIdx.x, blockIdx.x + gridDim.x, ...; item i = (tile i / nsplit, slice i % nsplit),
// whose columns are [slice * nkb / nsplit, (slice + 1) * nkb / nsplit).
struct UnitWalk {
    uint32_t item, tile, sp, kb, kb_end;
    __device__ __forceinline__ void set(uint32_t i, uint32_t nsplit, uint32_t nkb)
    {
        item = i;
        tile = i / nsplit;
        sp = i - tile * nsplit;
        kb = sp * nkb / nsplit;
        kb_end = (sp + 1) * nkb / nsplit;
    }
    __device__ __forceinline__ bool last() const { return kb + 1 == kb_end; }
    __device__ __forceinline__ void next(uint32_t nsplit, uint32_t nkb, uint32_t stride)
    {
        if (++kb == kb_end) set(item + stride, nsplit, nkb);
    }
};

}  // namespace wgb
