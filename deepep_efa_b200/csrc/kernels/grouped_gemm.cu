// Grouped expert GEMM for sm_100a: tcgen05.mma with the accumulator in TMEM, operands staged into
// 128-byte-swizzled shared memory by TMA (from this GPU's own memory only, never multicast), a
// persistent warp-specialised CTA per SM.
//
//   warp 0   : TMA producer   (one lane)  global -> smem ring, mbarrier complete_tx
//   warp 1   : MMA issuer     (one lane)  tcgen05.mma, tcgen05.commit frees smem stages and publishes
//                                         accumulator windows; also owns TMEM alloc / dealloc
//   warps 2.. : epilogue (4 warps for BF16, 8 for FP8)  tcgen05.ld -> registers -> (scale | SwiGLU) -> BF16 ->
//                                         per-warp smem transpose -> coalesced global stores
//
// A tile is 128 rows x kBlockN columns; a K block is 128 bytes per row (64 BF16 or 128 e4m3), i.e. one
// swizzle atom, consumed by four MMAs. Two accumulator windows in TMEM let the epilogue of window i
// overlap the MMAs of window i+1. BF16: a window is a whole output tile. FP8 with DeepSeek-style fp32
// scales (1x128 on activations, 128x128 on weights): a window is ONE K block; the epilogue multiplies it
// by scale_a[row, kb] * scale_b[nblock, kb] and accumulates in fp32 registers (the MMA's native block
// scaling wants power-of-two UE8M0 factors, which these scales are not).
//
// Every mbarrier wait is bounded; when a limit runs out the CTA raises a flag, all roles leave their
// loops, TMEM is released and the kernel returns.
//
// The reference has no GEMM: its users run their expert FFN between dispatch and combine themselves.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "gemm_api.h"
#include "prims.cuh"

namespace dx {

namespace {

constexpr int kBlockM = 128;
constexpr int kKBlockBytes = 128;      // one 128B swizzle atom per row
constexpr int kATileBytes = kBlockM * kKBlockBytes;  // 16 KiB
constexpr int kMaxGroups = 1024;

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait: returns false (and raises the CTA abort flag) when the limit runs out or another role
// has already aborted.
// `note` (optional, device memory) keeps the first wait that gave up: `what` = (role code << 56 | tile << 24 | k block << 8 | slot).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit,
                                          unsigned long long* note = nullptr, unsigned long long what = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            if (note != nullptr) atomicCAS(note, 0ull, what);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ unsigned long long wait_id(int role, int tile, int kb, int slot) {
    return ((unsigned long long)role << 56) | ((unsigned long long)(tile & 0xffffffff) << 24) | ((unsigned long long)(kb & 0xffff) << 8) |
           (unsigned long long)(slot & 0xff);
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <bool kFp8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kFp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in 128B-swizzled shared memory: rows are 128 bytes apart, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
    d |= (uint64_t)1 << 46;                        // descriptor version
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// MN-major operand tile (the tensor's contiguous dimension is the tile's row index, not K): the tile is stored as chunks of
// 64 rows; a chunk is 64 K-steps of 128 bytes (64 BF16 row elements), 128B-swizzled in groups of 8 K-steps. Stride byte
// offset = distance between 8-K-step groups (1024), leading byte offset = distance between 64-row chunks (8192).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(8192 >> 4) << 16;              // leading byte offset: next 64-row chunk
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: next group of 8 K-steps
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// Instruction descriptor: fp32 accumulate, M = 128, N = n; bit 15 / 16 = A / B is MN-major instead of K-major.
template <bool kFp8>
__device__ __forceinline__ uint32_t make_idesc(int n, int m = kBlockM, int a_mn = 0, int b_mn = 0) {
    uint32_t d = 0;
    d |= 1u << 4;                          // D format = F32
    d |= (kFp8 ? 0u : 1u) << 7;            // A format: E4M3 (f8f6f4) or BF16 (f16)
    d |= (kFp8 ? 0u : 1u) << 10;           // B format
    d |= (a_mn ? 1u : 0u) << 15;           // A major
    d |= (b_mn ? 1u : 0u) << 16;           // B major
    d |= (uint32_t)(n >> 3) << 17;         // N / 8
    d |= (uint32_t)(m >> 4) << 24;         // M / 16 (256 for a CTA pair)
    return d;
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one 256-row MMA; each stages its own 128 rows of A and HALF
// of the B tile, so the bytes every SM pulls from L2 per FLOP drop by a third. No load here is a multicast: each CTA's TMA
// writes only its own shared memory and signals the leader CTA's mbarrier.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t bar_cluster_addr, void* dst, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
template <bool kFp8>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kFp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// ---- native block scaling (kind::mxf8f6f4.block_scale): UE8M0 scale factors live in TMEM, one byte per 32 K-elements and
// row. A 128-row x 128-K scale tile is a 512-byte atom in shared memory: the byte of row (m0 + 32*m1), K sub-block kb sits at
// m0*16 + m1*4 + kb; tcgen05.cp moves it to four TMEM columns (lane m0, column m1, byte kb), replicated to all four lane
// quarters. With one scale per 128 K-elements the four bytes of a word are equal.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// 32 rows of 16 bytes, contiguous: no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset (one 16-byte column only)
    d |= (uint64_t)(128 >> 4) << 32;   // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version
    return d;                          // layout type 0: no swizzle
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// Instruction descriptor of the block-scaled kind: E4M3 operands (format 0), K-major, UE8M0 scales, scale-factor ids 0.
__device__ __forceinline__ uint32_t make_idesc_mx(int n, int m = kBlockM) {
    uint32_t d = 0;
    d |= (uint32_t)(n >> 3) << 17;         // N / 8
    d |= 1u << 23;                         // scale format: E8M0
    d |= (uint32_t)(m >> 4) << 24;         // M / 16 (256 for a CTA pair)
    return d;
}
// CTA-pair forms: one instruction makes BOTH CTAs copy their own scale atoms (same shared-memory offset) into their own TMEM,
// and one MMA covers the 256 rows of the pair; every CTA holds the scale factors of its own 128 rows of A and of ALL columns.
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mx_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Orders what this thread observed through ordinary loads (the arrival counter) before its later TMA reads of the rows.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ int4 pack8_bf16(const float* o) {
    int4 w;
    __nv_bfloat162 t0 = __floats2bfloat162_rn(o[0], o[1]), t1 = __floats2bfloat162_rn(o[2], o[3]);
    __nv_bfloat162 t2 = __floats2bfloat162_rn(o[4], o[5]), t3 = __floats2bfloat162_rn(o[6], o[7]);
    w.x = *reinterpret_cast<int*>(&t0);
    w.y = *reinterpret_cast<int*>(&t1);
    w.z = *reinterpret_cast<int*>(&t2);
    w.w = *reinterpret_cast<int*>(&t3);
    return w;
}

// Stores a 32-row x kCols BF16 block that a warp holds one row per lane. Writing it straight from registers would put
// every lane on its own 32-byte sector (half filled); instead the block is transposed through a per-warp shared
// buffer (XOR-swizzled 16-byte pieces) so that each store instruction covers whole rows: 128 contiguous bytes per row
// for kCols = 64, 64 bytes for kCols = 32.
template <int kCols>
__device__ __forceinline__ void store_block_coalesced(int4* stage, const int4 (&regs)[kCols / 8], __nv_bfloat16* gbase, int ldc,
                                                      int rows_valid, int lane) {
    constexpr int P = kCols / 8;    // 16-byte pieces per row
    constexpr int RPI = 32 / P;     // rows covered by one store instruction
    __syncwarp();
#pragma unroll
    for (int j = 0; j < P; ++j) stage[lane * P + (j ^ (lane & (P - 1)))] = regs[j];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < P; ++i) {
        const int row = i * RPI + lane / P, piece = lane % P;
        const int4 v = stage[row * P + (piece ^ (row & (P - 1)))];
        if (row < rows_valid) *reinterpret_cast<int4*>(gbase + (size_t)row * ldc + piece * 8) = v;
    }
}

// Same block, but every row goes to its own destination: lane l holds the address of row l (nullptr = drop the row).
template <int kCols>
__device__ __forceinline__ void store_block_scattered(int4* stage, const int4 (&regs)[kCols / 8], __nv_bfloat16* my_row_ptr, int lane) {
    constexpr int P = kCols / 8;
    constexpr int RPI = 32 / P;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < P; ++j) stage[lane * P + (j ^ (lane & (P - 1)))] = regs[j];
    __syncwarp();
    const unsigned long long mine = reinterpret_cast<unsigned long long>(my_row_ptr);
#pragma unroll
    for (int i = 0; i < P; ++i) {
        const int row = i * RPI + lane / P, piece = lane % P;
        const int4 v = stage[row * P + (piece ^ (row & (P - 1)))];
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, mine, row));
        if (dst != nullptr) *reinterpret_cast<int4*>(dst + piece * 8) = v;
    }
}

// 32 rows x 256 bytes: lane l holds row l as 16 pieces of 16 bytes, and the row's destination (nullptr = drop the row). Eight rows at a
// time pass through a 2 KiB staging buffer (XOR-swizzled pieces), so that every store instruction covers two whole 256-byte rows:
// rows that leave for another GPU cross NVLink in 256-byte packets.
__device__ __forceinline__ void store_rows_256(int4* stage, const int4 (&regs)[16], __nv_bfloat16* my_row_ptr, int lane) {
    const unsigned long long mine = reinterpret_cast<unsigned long long>(my_row_ptr);
#pragma unroll
    for (int g8 = 0; g8 < 4; ++g8) {
        __syncwarp();
        if ((lane >> 3) == g8) {
#pragma unroll
            for (int j = 0; j < 16; ++j) stage[(lane & 7) * 16 + (j ^ (lane & 7))] = regs[j];
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r8 = i * 2 + (lane >> 4), piece = lane & 15;
            const int4 v = stage[r8 * 16 + (piece ^ r8)];
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, mine, g8 * 8 + r8));
            if (dst != nullptr) *reinterpret_cast<int4*>(dst + piece * 8) = v;
        }
    }
}

struct TileInfo {
    int a_row, a_k0, b_row, b_row2, b_k0, num_kb, c_row, c_col, group, nblock, nblock2;
    int c_row_end;  // first output row this tile must not write (end of its group; groups need no 128-row alignment)
    int nt;         // n-tile index inside the group (kMx: selects the B scale atoms)
    // MN-major operands: first tile row inside the tensor's contiguous dimension, and the tensor row of K index 0
    int a_mn0, a_kbase, b_mn0, b_kbase;
};

// kRowScatter: the scatter epilogue writes every output row of a 128-column tile as ONE 256-byte piece (the largest NVLink
// packet) instead of two 128-byte pieces; it needs an 8 KiB staging buffer per epilogue warp and gives up one pipeline stage.
template <int kBlockN, bool kFp8, bool kSwiGLU, bool kPair, bool kMx = false, bool kRowScatter = false>
struct Cfg {
    static constexpr bool kPromote = kFp8 && !kMx;  // FP8 with fp32 scales: every K block is promoted on the CUDA cores
    static constexpr int kSfBAtoms = kBlockN / 128;                  // 512-byte scale atoms of the B tile
    static constexpr int kSfTxBytes = kMx ? 512 * (1 + kSfBAtoms) : 0;   // per stage: scale atoms of A and of B
    static constexpr int kSfBytes = (kSfTxBytes + 1023) / 1024 * 1024;   // stages stay 1024-byte aligned (swizzle atoms)
    // B rows staged per CTA: a CTA pair splits the tile's N between its two CTAs
    static constexpr int kBRows = kPair ? kBlockN / 2 : kBlockN;
    static constexpr int kBTileBytes = kBRows * kKBlockBytes;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes + kSfBytes;
    static constexpr int kStageTxBytes = kATileBytes + kBTileBytes + kSfTxBytes;  // bytes the copies of one stage deliver
    static constexpr int kStages = kMx ? ((kBlockN == 256) ? (kPair ? 5 : 4) : (kRowScatter ? 5 : 6)) : kPair ? ((kBlockN == 256) ? (kFp8 ? 5 : 6) : (kFp8 ? 6 : 8)) : ((kBlockN == 256) ? 4 : (kFp8 ? 5 : 6));
    static constexpr int kTileRows = kPair ? 2 * kBlockM : kBlockM;  // rows of one scheduled tile (both CTAs of a pair)
    // Accumulator windows in TMEM. FP8 hands the epilogue one window per K block, so the MMA warp needs to run several
    // K blocks ahead of the promotion: four 128-column windows fill TMEM. BF16 hands over one window per tile: two.
    // kMx with 256-column tiles: ONE window (two would fill TMEM and leave no room for the scale columns); the epilogue of
    // that variant drains the accumulator into registers first and releases the window before it stores.
    static constexpr int kWindows = kPromote ? 4 : ((kMx && kBlockN == 256) ? 1 : 2);
    static constexpr int kSfCol0 = kWindows * kBlockN;   // kMx: two alternating sets of (4 columns A + 4 per B atom) after the windows
    static constexpr int kSfColsPerBuf = 4 + 4 * kSfBAtoms;
    static constexpr int kTmemCols = kMx ? 512 : kWindows * kBlockN;
    static constexpr int kOutCols = kSwiGLU ? kBlockN / 2 : kBlockN;
    // FP8 promotes every K block on the CUDA cores, so it gets two epilogue warps per TMEM lane quarter (each takes half
    // of the columns); BF16 reads the accumulator once per tile and one warp per quarter is plenty.
    // The single-window wide tile also gets two warps per quarter: each drains half of the columns RAW (128 fp32 registers per
    // thread) and hands the window back at once, so the MMA issuer idles for the TMEM reads only, not for the SwiGLU arithmetic.
    static constexpr bool kSplitDrain = kMx && kBlockN == 256;
    static constexpr int kEpiWarps = (kPromote || kSplitDrain) ? 8 : 4;
    static constexpr int kThreads = 64 + 32 * kEpiWarps;
    static constexpr int kOutStageBytes = kRowScatter ? 8192 : (kSplitDrain ? 2048 : 4096);    // per epilogue warp: 32 rows x 32 / 64 (128) BF16
    // kSplitDrain with quantised output: the two warps of a quarter exchange their half-row maxima here (two tile parities)
    static constexpr int kXchBytes = kSplitDrain ? 2 * 2 * kBlockM * 8 : 0;
    static constexpr size_t kSmemBytes =
        (size_t)kStages * kStageBytes + (size_t)kEpiWarps * kOutStageBytes + 1024 /*align*/ + 256 /*barriers*/ + (kMaxGroups + 1) * 4 + kXchBytes;
};

template <int kBlockN, bool kFp8, bool kSwiGLU, bool kPair, bool kMx = false, bool kRowScatter = false>
__global__ void __launch_bounds__((Cfg<kBlockN, kFp8, kSwiGLU, kPair, kMx, kRowScatter>::kThreads), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb, const GroupedGemmArgs p) {
    using C = Cfg<kBlockN, kFp8, kSwiGLU, kPair, kMx, kRowScatter>;
    static_assert(!kRowScatter || (kMx && !kSwiGLU && !kPair && kBlockN == 128), "whole-row scatter: natively block-scaled 128-column tiles");
    static_assert(!kMx || (kFp8 && ((!kPair && kBlockN == 128) || (kBlockN == 256 && (kSwiGLU || !kPair)))),
                  "native block scaling: e4m3 operands; 128-column tiles, 256-column tiles, or 256-column SwiGLU tiles on a CTA pair");
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;   // 0 = leader (issues the MMAs of the pair)
    const int sched_id = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int sched_stride = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint8_t* out_stage_base = smem + (size_t)C::kStages * C::kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage_base + (size_t)C::kEpiWarps * C::kOutStageBytes);
    uint64_t* full = bars;                       // [kStages]
    uint64_t* empty = bars + C::kStages;         // [kStages]
    uint64_t* tmem_full = bars + 2 * C::kStages; // [kWindows]
    uint64_t* tmem_empty = tmem_full + C::kWindows;  // [kWindows]
    int* tile_start = reinterpret_cast<int*>(bars + 32);  // [G+1] first tile index of every group
    volatile unsigned long long* xch = reinterpret_cast<volatile unsigned long long*>(bars + 32 + (kMaxGroups + 2) / 2);  // [2][2][kBlockM] (tile tag << 32 | amax bits)
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ volatile int s_prod_state[2];  // what the loader is doing (1 = arrival gate, 2 = free stage, 3 = loads issued) and for which tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.num_groups;
    const int elem_per_kb = kFp8 ? 128 : 64;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < C::kWindows; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], kPair ? 2 * C::kEpiWarps : C::kEpiWarps);  // the leader collects both CTAs' epilogue warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
        // tile table
        int run = 0;
        const int tiles_n = p.mode == 0 ? p.n / kBlockN : 0;
        const int tiles_fixed = p.mode == 1 ? ((p.n + C::kTileRows - 1) / C::kTileRows) * (p.k / kBlockN) : 0;
        for (int g = 0; g < G; ++g) {
            tile_start[g] = run;
            // native block scaling reads one scale atom per 128-row tile, so a group that does not start on a tile boundary
            // would be scaled with its neighbour's factors: flag it (value 2) instead of returning silently wrong numbers
            if (kMx && (p.m_offsets[g] & 127) != 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 2);
            if (p.mode == 0) {
                const int rows = (p.m_ends != nullptr ? p.m_ends[g] : p.m_offsets[g + 1]) - p.m_offsets[g];
                run += ((max(rows, 0) + C::kTileRows - 1) / C::kTileRows) * tiles_n;
            } else {
                run += tiles_fixed;
            }
        }
        tile_start[G] = run;
    }
    if constexpr (C::kSplitDrain) {
        for (int i = threadIdx.x; i < C::kXchBytes / 8; i += C::kThreads) xch[i] = 0ull;
    }
    if (warp == 1) {
        if constexpr (kPair) tmem_alloc_pair(&s_tmem_base, C::kTmemCols);
        else tmem_alloc(&s_tmem_base, C::kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const int total_tiles = tile_start[G];
    volatile int* abort_flag = &s_abort;
    const long long limit = p.timeout_cycles;
    unsigned long long* note = p.trace != nullptr ? p.trace + 2 : nullptr;  // trace[2]: first bounded wait that gave up

    // Decodes tile index -> coordinates; `g` is a cursor that only moves forward.
    auto decode = [&](int tile, int& g, TileInfo& ti) {
        while (tile >= tile_start[g + 1]) ++g;
        const int local = tile - tile_start[g];
        const int m0 = p.m_offsets[g], m1 = (p.mode == 0 && p.m_ends != nullptr) ? max(p.m_ends[g], m0) : p.m_offsets[g + 1];
        ti.group = g;
        if (p.mode == 0) {
            const int tiles_m = (m1 - m0 + C::kTileRows - 1) / C::kTileRows;
            const int tiles_n_ = p.n / kBlockN;
            // order 0: consecutive tiles share the weight tile (n outer); order 1: they share the activation tile (m outer)
            const int nt = p.tile_order == 0 ? local / tiles_m : local % tiles_n_;
            const int mt = p.tile_order == 0 ? local % tiles_m : local / tiles_n_;
            ti.a_row = m0 + mt * C::kTileRows + (int)cta_rank * kBlockM;
            ti.nt = nt;
            ti.a_mn0 = ti.a_kbase = 0;                                          // mode 0: A is always K-major
            ti.b_mn0 = nt * kBlockN + (int)cta_rank * (kBlockN / 2);            // MN-major B: [G * K, N], N contiguous
            ti.b_kbase = g * p.k;
            ti.a_k0 = 0;
            ti.b_k0 = 0;
            ti.num_kb = p.k / elem_per_kb;
            ti.c_row = ti.a_row;
            ti.c_row_end = min(m1, p.m_total);
            if (kSwiGLU) {
                const int half = kBlockN / 2, inter = p.n / 2;
                ti.b_row = g * p.n + nt * half;            // gate rows
                ti.b_row2 = g * p.n + inter + nt * half;   // up rows
                ti.c_col = nt * half;
                ti.nblock = (nt * half) / 128;
                ti.nblock2 = (inter + nt * half) / 128;
            } else {
                ti.b_row = g * p.n + nt * kBlockN + (int)cta_rank * (kBlockN / 2);  // a pair splits the tile's N
                ti.b_row2 = 0;
                ti.c_col = nt * kBlockN;
                ti.nblock = (nt * kBlockN) / 128;
                ti.nblock2 = ti.nblock;
            }
        } else {
            const int tiles_j = p.k / kBlockN;
            const int it = local / tiles_j, jt = local % tiles_j;
            ti.a_row = it * C::kTileRows + (int)cta_rank * kBlockM;
            ti.b_row = jt * kBlockN + (int)cta_rank * (kBlockN / 2);
            ti.b_row2 = 0;
            ti.a_mn0 = ti.a_row;                                                // MN-major: A is [M, N_out], B is [M, K_out]
            ti.b_mn0 = ti.b_row;
            ti.a_kbase = ti.b_kbase = m0;
            ti.a_k0 = m0;
            ti.b_k0 = m0;
            ti.num_kb = (m1 - m0) / elem_per_kb;
            ti.c_row = g * p.n + ti.a_row;
            ti.c_row_end = min((g + 1) * p.n, p.num_groups * p.n);
            ti.c_col = jt * kBlockN;
            ti.nblock = ti.nblock2 = 0;
        }
    };

    // An epilogue warp hands an accumulator window back to the MMA issuer: in a pair that is the leader CTA's barrier.
    auto release_window = [&](uint64_t* bar) {
        if constexpr (kPair) {
            if (cta_rank == 0) mbar_arrive(bar);
            else mbar_arrive_cluster(mapa_shared(smem_u32(bar), 0));
        } else {
            mbar_arrive(bar);
        }
    };

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int stage = 0, phase = 0, g = 0;
            int issued = 0;  // stages armed so far (saturating), for the drain on the abort path
            int gated_group = -1;
            bool stamped = false;
            TileInfo ti;
            bool ok = true;
            for (int tile = sched_id; tile < total_tiles && ok; tile += sched_stride) {
                decode(tile, g, ti);
                s_prod_state[1] = tile;
                if (p.ready != nullptr && ti.group != gated_group) {
                    s_prod_state[0] = 1;
                    // the rows of this group come from other GPUs: wait until all of them have landed
                    const unsigned long long want = p.expected[ti.group];
                    if (ld_acquire_sys_u64(p.ready + ti.group) < want) {
                        const long long t0 = clock64();
                        while (ld_acquire_sys_u64(p.ready + ti.group) < want) {
                            if (*abort_flag || clock64() - t0 > limit) {
                                if (!*abort_flag && note != nullptr) atomicCAS(note, 0ull, wait_id(2, tile, 0, ti.group));
                                *abort_flag = 1;
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
                    fence_proxy_async();
                    gated_group = ti.group;
                }
                if (p.trace != nullptr && !stamped) {
                    atomicMin(&p.trace[0], global_timer_ns());
                    stamped = true;
                }
                for (int kb = 0; kb < ti.num_kb; ++kb) {
                    s_prod_state[0] = 2;
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, limit, note, wait_id(1, tile, kb, stage))) {
                        ok = false;
                        break;
                    }
                    uint8_t* sa = stage_base + (size_t)stage * C::kStageBytes;
                    uint8_t* sb = sa + kATileBytes;
                    if constexpr (kPair) {
                        // both CTAs fill their own stage and signal the LEADER's barrier, which expects the bytes of both
                        const uint32_t leader_full = mapa_shared(smem_u32(&full[stage]), 0);
                        if (cta_rank == 0) mbar_expect_tx(&full[stage], 2 * C::kStageTxBytes);
                        tma_load_2d_pair(&map_a, leader_full, sa, ti.a_k0 + kb * elem_per_kb, ti.a_row);
                        tma_load_2d_pair(&map_b, leader_full, sb, ti.b_k0 + kb * elem_per_kb,
                                         (kSwiGLU && cta_rank == 1) ? ti.b_row2 : ti.b_row);  // SwiGLU: gate half / up half
                        if constexpr (kMx) {
                            // scale atoms as rows of 32-bit words: this CTA's own 128 rows of A, and the whole tile's B columns
                            uint8_t* ssf = sb + C::kBTileBytes;
                            const int nkb = p.k / 128;
                            tma_load_2d_pair(&map_sfa, leader_full, ssf, 0, (ti.a_row >> 7) * nkb + kb);
                            tma_load_2d_pair(&map_sfb, leader_full, ssf + 512, 0, (ti.group * (p.n / kBlockN) + ti.nt) * nkb + kb);
                        }
                        if (issued < C::kStages) ++issued;
                        if (++stage == C::kStages) {
                            stage = 0;
                            phase ^= 1;
                        }
                        continue;
                    }
                    s_prod_state[0] = 3;
                    mbar_expect_tx(&full[stage], C::kStageTxBytes);
                    if constexpr (kMx) {
                        // scale atoms: [row tile][K block][512] for A, [group][n tile][K block][512] for B
                        uint8_t* ssf = sb + C::kBTileBytes;
                        const size_t nkb = (size_t)(p.k / 128);
                        bulk_load_1d(ssf, p.sfa_atoms + ((size_t)(ti.a_row >> 7) * nkb + kb) * 512, 512, &full[stage]);
                        bulk_load_1d(ssf + 512, p.sfb_atoms + (((size_t)ti.group * (p.n / kBlockN) + ti.nt) * nkb + kb) * (512 * C::kSfBAtoms),
                                     512 * C::kSfBAtoms, &full[stage]);
                    }
                    if constexpr (!kFp8 && !kSwiGLU && !kMx) {
                        if (p.a_mn | p.b_mn) {
                            // an MN-major tile arrives as chunks of 64 rows x 64 K-steps (8 KiB each)
                            if (p.a_mn) {
#pragma unroll
                                for (int j = 0; j < kBlockM / 64; ++j)
                                    tma_load_2d(&map_a, &full[stage], sa + j * 8192, ti.a_mn0 + j * 64, ti.a_kbase + kb * 64);
                            } else {
                                tma_load_2d(&map_a, &full[stage], sa, ti.a_k0 + kb * elem_per_kb, ti.a_row);
                            }
                            if (p.b_mn) {
#pragma unroll
                                for (int j = 0; j < kBlockN / 64; ++j)
                                    tma_load_2d(&map_b, &full[stage], sb + j * 8192, ti.b_mn0 + j * 64, ti.b_kbase + kb * 64);
                            } else {
                                tma_load_2d(&map_b, &full[stage], sb, ti.b_k0 + kb * elem_per_kb, ti.b_row);
                            }
                            if (issued < C::kStages) ++issued;
                            if (++stage == C::kStages) {
                                stage = 0;
                                phase ^= 1;
                            }
                            continue;
                        }
                    }
                    tma_load_2d(&map_a, &full[stage], sa, ti.a_k0 + kb * elem_per_kb, ti.a_row);
                    if (kSwiGLU) {
                        tma_load_2d(&map_b, &full[stage], sb, ti.b_k0 + kb * elem_per_kb, ti.b_row);
                        tma_load_2d(&map_b, &full[stage], sb + C::kBTileBytes / 2, ti.b_k0 + kb * elem_per_kb, ti.b_row2);
                    } else {
                        tma_load_2d(&map_b, &full[stage], sb, ti.b_k0 + kb * elem_per_kb, ti.b_row);
                    }
                    if (issued < C::kStages) ++issued;
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            // Own copies in flight land in this CTA's shared memory: before the CTA may exit, wait (bounded) for every stage
            // that was armed but whose completion this lane has not yet seen. `stage`/`phase` point at the next stage to
            // fill, so the kStages stages before it are the candidates, each with the phase it was armed in.
            if (!ok) {
                if (kPair && cta_rank == 1) {
                    // the peer's copies signal the leader's barriers, which this CTA cannot poll: give them a fixed grace time
                    const long long t0 = clock64();
                    while (clock64() - t0 < 400000) {
                    }
                } else {
                    int st = stage, ph = phase;
                    for (int i = 0; i < C::kStages && i < issued; ++i) {
                        if (--st < 0) {
                            st = C::kStages - 1;
                            ph ^= 1;
                        }
                        const long long t0 = clock64();
                        while (!mbar_try_wait(&full[st], ph) && clock64() - t0 < limit) {
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0 && cta_rank == 0) {
            const uint32_t idesc = kMx ? make_idesc_mx(kBlockN, C::kTileRows) : make_idesc<kFp8>(kBlockN, C::kTileRows, p.a_mn, p.b_mn);
            // bytes (in 16-byte units) one K = 16 step moves the operand's start address: 32 B inside the swizzle atom when K
            // is contiguous, 16 K-steps of 128 B when the rows are
            const uint64_t a_kstep = p.a_mn ? 128 : 2, b_kstep = p.b_mn ? 128 : 2;
            int sf_buf = 0;
            int stage = 0, phase = 0, g = 0;
            int win = 0, win_phase = 0;  // accumulator window ring
            TileInfo ti;
            bool ok = true;
            for (int tile = sched_id; tile < total_tiles && ok; tile += sched_stride) {
                decode(tile, g, ti);
                if (ti.num_kb == 0) continue;  // epilogue writes zeros on its own
                for (int kb = 0; kb < ti.num_kb; ++kb) {
                    const bool new_window = C::kPromote ? true : (kb == 0);
                    if (new_window) {
                        if (!mbar_wait(&tmem_empty[win], win_phase ^ 1, abort_flag, limit, note, wait_id(3, tile, kb, win))) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                    }
                    if (!mbar_wait(&full[stage], phase, abort_flag, limit, note, wait_id(4, tile, kb, stage))) {
                        if (note != nullptr) atomicCAS(note + 1, 0ull, ((unsigned long long)s_prod_state[0] << 32) | (unsigned)s_prod_state[1]);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage_base + (size_t)stage * C::kStageBytes);
                    const uint32_t sb = sa + kATileBytes;
                    const uint64_t adesc = p.a_mn ? make_smem_desc_mn(sa) : make_smem_desc(sa);
                    const uint64_t bdesc = p.b_mn ? make_smem_desc_mn(sb) : make_smem_desc(sb);
                    const uint32_t tmem_d = tmem_base + (uint32_t)(win * kBlockN);
                    if constexpr (kMx) {
                        // scale atoms of this stage -> TMEM (alternating column sets), then four K=32 MMAs that read them
                        const uint32_t ssf = sb + C::kBTileBytes;
                        const uint32_t t_sfa = tmem_base + (uint32_t)(C::kSfCol0 + sf_buf * C::kSfColsPerBuf), t_sfb = t_sfa + 4;
                        if constexpr (kPair) {
                            tmem_cp_sf_pair(t_sfa, make_sf_desc(ssf));
#pragma unroll
                            for (int at = 0; at < C::kSfBAtoms; ++at) tmem_cp_sf_pair(t_sfb + 4 * at, make_sf_desc(ssf + 512 + 512 * at));
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                umma_mx_pair(tmem_d, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, t_sfa, t_sfb,
                                             (new_window && j == 0) ? 0u : 1u);
                        } else {
                            tmem_cp_sf(t_sfa, make_sf_desc(ssf));
#pragma unroll
                            for (int at = 0; at < C::kSfBAtoms; ++at) tmem_cp_sf(t_sfb + 4 * at, make_sf_desc(ssf + 512 + 512 * at));
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                umma_mx(tmem_d, adesc + (uint64_t)(j * 2), bdesc + (uint64_t)(j * 2), idesc, t_sfa, t_sfb,
                                        (new_window && j == 0) ? 0u : 1u);
                        }
                        sf_buf ^= 1;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // +32 bytes along K inside the swizzle atom = +2 in the 16-byte start-address field
                            if constexpr (kPair)
                                umma_pair<kFp8>(tmem_d, adesc + (uint64_t)j * a_kstep, bdesc + (uint64_t)j * b_kstep, idesc,
                                                (new_window && j == 0) ? 0u : 1u);
                            else
                                umma<kFp8>(tmem_d, adesc + (uint64_t)j * a_kstep, bdesc + (uint64_t)j * b_kstep, idesc,
                                           (new_window && j == 0) ? 0u : 1u);
                        }
                    }
                    // smem stage reusable once these MMAs have read it (in both CTAs of a pair)
                    if constexpr (kPair) {
                        umma_commit_pair(smem_u32(&empty[stage]));
                        umma_commit_pair(mapa_shared(smem_u32(&empty[stage]), 1));
                    } else {
                        umma_commit(&empty[stage]);
                    }
                    const bool window_done = C::kPromote ? true : (kb == ti.num_kb - 1);
                    if (window_done) {
                        if constexpr (kPair) {
                            umma_commit_pair(smem_u32(&tmem_full[win]));
                            umma_commit_pair(mapa_shared(smem_u32(&tmem_full[win]), 1));
                        } else {
                            umma_commit(&tmem_full[win]);
                        }
                        if (++win == C::kWindows) {
                            win = 0;
                            win_phase ^= 1;
                        }
                    }
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        // ================= epilogue =================
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;          // FP8 only: which half of the columns this warp promotes
        const int row_in_tile = q * 32 + lane;
        int4* out_stage = reinterpret_cast<int4*>(out_stage_base + (size_t)(warp - 2) * C::kOutStageBytes);
        int g = 0, win = 0, win_phase = 0;
        int xch_iter = 0;  // split drain: tiles whose row maxima went through the exchange so far
        (void)xch_iter;
        TileInfo ti;
        bool ok = true;
        __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(p.c);
        const int ldc = p.mode == 0 ? (kSwiGLU ? p.n / 2 : p.n) : p.k;
        const bool scatter = !kSwiGLU && p.mode == 0 && p.row_info != nullptr;
        for (int tile = sched_id; tile < total_tiles && ok; tile += sched_stride) {
            decode(tile, g, ti);
            const int row = ti.c_row + row_in_tile;
            __nv_bfloat16* crow = cbase + (size_t)row * ldc + ti.c_col;
            // scatter epilogue: this lane's row goes to row (word & 0xffffff) of the matrix at scatter_bases[word >> 24]
            __nv_bfloat16* scat_ptr = nullptr;
            if (scatter && row < ti.c_row_end) {
                const int word = p.row_info[row];
                if (word >= 0)
                    scat_ptr = reinterpret_cast<__nv_bfloat16*>(p.scatter_bases[word >> 24]) + (size_t)(word & 0xffffff) * ldc + ti.c_col;
            }
            if (ti.num_kb == 0) {
                __nv_bfloat16* zrow = scatter ? scat_ptr : crow;
                if (row < ti.c_row_end && half == 0 && zrow != nullptr)
                    for (int c = 0; c < C::kOutCols; c += 8) *reinterpret_cast<int4*>(zrow + c) = make_int4(0, 0, 0, 0);
                continue;
            }
            if constexpr (C::kPromote) {
                // One window per K block, promoted into fp32 registers with the two scales. A warp owns two 32-column
                // chunks: with SwiGLU a gate chunk and the matching up chunk, otherwise two neighbouring chunks.
                constexpr int kLo0 = 0, kHalfCols = kBlockN / 2;
                const int c_lo = kSwiGLU ? half * 32 : half * kHalfCols;
                const int c_hi = kSwiGLU ? kHalfCols + half * 32 : half * kHalfCols + 32;
                (void)kLo0;
                float acc[64];
#pragma unroll
                for (int i = 0; i < 64; ++i) acc[i] = 0.f;
                const int num_kscales = p.k / 128;
                const int n_blocks = p.n / 128;
                const float* sa_row = p.a_scales + (size_t)min(row, p.m_total - 1) * num_kscales;
                const float* sb0 = p.b_scales + ((size_t)ti.group * n_blocks + ti.nblock) * num_kscales;
                const float* sb1 = p.b_scales + ((size_t)ti.group * n_blocks + ti.nblock2) * num_kscales;
                // A warp whose 32 rows all lie past the end of the group (masked low-latency layout: a handful of valid rows
                // per expert) only keeps the window ring moving; it promotes nothing.
                const bool warp_has_rows = ti.c_row + q * 32 < ti.c_row_end;
                for (int kb = 0; kb < ti.num_kb; ++kb) {
                    if (!warp_has_rows) {
                        if (!mbar_wait(&tmem_full[win], win_phase, abort_flag, limit, note, wait_id(7, tile, kb, warp))) {
                            ok = false;
                            break;
                        }
                        __syncwarp();
                        if (lane == 0) release_window(&tmem_empty[win]);
                        if (++win == C::kWindows) {
                            win = 0;
                            win_phase ^= 1;
                        }
                        continue;
                    }
                    // Ungated: the activation scale is fetched ahead of the wait, to hide its latency. With arrival gating the
                    // scales are written by other GPUs during this kernel, and only the accumulator hand-over orders this warp
                    // after the loader's acquire of the group's arrival counter: the load has to come after the wait (L2 only).
                    float sa = 0.f;
                    if (p.ready == nullptr) sa = __ldcg(sa_row + kb);
                    const float wb0 = __ldg(sb0 + kb), wb1 = kSwiGLU ? __ldg(sb1 + kb) : 0.f;
                    if (!mbar_wait(&tmem_full[win], win_phase, abort_flag, limit, note, wait_id(5, tile, kb, warp))) {
                        ok = false;
                        break;
                    }
                    if (p.ready != nullptr) sa = __ldcg(sa_row + kb);
                    const float s_lo = sa * wb0, s_hi = kSwiGLU ? sa * wb1 : s_lo;
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(win * kBlockN);
                    uint32_t v[32], u[32];
                    tmem_ld32(taddr + c_lo, v);
                    tmem_ld32(taddr + c_hi, u);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_window(&tmem_empty[win]);  // the window is free as soon as it sits in registers
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        acc[i] = fmaf(__uint_as_float(v[i]), s_lo, acc[i]);
                        acc[32 + i] = fmaf(__uint_as_float(u[i]), s_hi, acc[32 + i]);
                    }
                    if (++win == C::kWindows) {
                        win = 0;
                        win_phase ^= 1;
                    }
                }
                if (!ok) break;
                {
                    // rows of this warp: ti.c_row + q*32 .. +32; the block base is row 0 of the warp
                    __nv_bfloat16* wbase = cbase + (size_t)(ti.c_row + q * 32) * ldc + ti.c_col;
                    const int rows_valid = min(32, ti.c_row_end - (ti.c_row + q * 32));
                    if constexpr (kSwiGLU) {
                        int4 regs[4];
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) o[i] = silu(acc[c + i]) * acc[32 + c + i];
                            regs[c / 8] = pack8_bf16(o);
                        }
                        store_block_coalesced<32>(out_stage, regs, wbase + half * 32, ldc, rows_valid, lane);
                    } else {
                        int4 regs[8];
#pragma unroll
                        for (int c = 0; c < 64; c += 8) regs[c / 8] = pack8_bf16(&acc[c]);
                        if (scatter) store_block_scattered<64>(out_stage, regs, scat_ptr != nullptr ? scat_ptr + half * kHalfCols : nullptr, lane);
                        else store_block_coalesced<64>(out_stage, regs, wbase + half * kHalfCols, ldc, rows_valid, lane);
                    }
                }
            } else {
                if (!mbar_wait(&tmem_full[win], win_phase, abort_flag, limit, note, wait_id(6, tile, 0, warp))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(win * kBlockN);
                __nv_bfloat16* wbase = cbase + (size_t)(ti.c_row + q * 32) * ldc + ti.c_col;
                const int rows_valid = min(32, ti.c_row_end - (ti.c_row + q * 32));
                if constexpr (kSwiGLU && C::kWindows == 1) {
                    // Single window, two warps per lane quarter: this warp takes 64 of the tile's 128 output columns. Their gate
                    // and up accumulators go to registers raw, the window returns to the MMA issuer right away, and the
                    // arithmetic and the stores run while the next tile accumulates.
                    uint32_t v[2][32], u[2][32];
                    tmem_ld32(taddr + half * 64, v[0]);
                    tmem_ld32(taddr + half * 64 + 32, v[1]);
                    tmem_ld32(taddr + kBlockN / 2 + half * 64, u[0]);
                    tmem_ld32(taddr + kBlockN / 2 + half * 64 + 32, u[1]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_window(&tmem_empty[win]);
                    int4 keep[2][4];
#pragma unroll
                    for (int ci = 0; ci < 2; ++ci)
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float o[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[j] = silu(__uint_as_float(v[ci][i + j])) * __uint_as_float(u[ci][i + j]);
                            keep[ci][i / 8] = pack8_bf16(o);
                        }
                    if constexpr (kMx) {
                        if (p.c_fp8 != nullptr) {
                            // The tile's 128 output columns are exactly one scale block of the next GEMM's activation operand: quantise
                            // here (same arithmetic as the standalone cast applied to the BF16 values: power-of-two scale from the
                            // row's amax) and write e4m3 + the UE8M0 atom word. The row's other 64 columns sit in the partner warp
                            // of this quarter; the two exchange their maxima through shared memory, tagged with the tile number.
                            float amax = 0.f;
#pragma unroll
                            for (int ci = 0; ci < 2; ++ci)
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const int4 v4 = keep[ci][j];
                                    const uint32_t w4[4] = {(uint32_t)v4.x, (uint32_t)v4.y, (uint32_t)v4.z, (uint32_t)v4.w};
#pragma unroll
                                    for (int t = 0; t < 4; ++t) {
                                        const float2 f = bf16x2_to_f2(w4[t]);
                                        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                                    }
                                }
                            const int par = xch_iter & 1;
                            ++xch_iter;
                            const unsigned tag = (unsigned)tile + 1u;
                            xch[(par * 2 + half) * kBlockM + row_in_tile] = ((unsigned long long)tag << 32) | __float_as_uint(amax);
                            volatile unsigned long long* other = xch + (par * 2 + (half ^ 1)) * kBlockM + row_in_tile;
                            unsigned long long w = *other;
                            if ((unsigned)(w >> 32) != tag) {
                                const long long t0 = clock64();
                                while ((unsigned)((w = *other) >> 32) != tag) {
                                    if (*abort_flag || clock64() - t0 > limit) {
                                        if (!*abort_flag && note != nullptr) atomicCAS(note, 0ull, wait_id(7, tile, 0, warp));
                                        *abort_flag = 1;
                                        ok = false;
                                        break;
                                    }
                                }
                            }
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                            amax = fmaxf(amax, __uint_as_float((unsigned)w));
                            float scale, inv;
                            fp8_scale_from_amax(amax, true, scale, inv);
                            int4 q8[4];
#pragma unroll
                            for (int ci = 0; ci < 2; ++ci)
#pragma unroll
                                for (int jj = 0; jj < 2; ++jj) {
                                    uint32_t outw[4];
#pragma unroll
                                    for (int h2 = 0; h2 < 2; ++h2) {
                                        const int4 v4 = keep[ci][jj * 2 + h2];
                                        const float2 f0 = bf16x2_to_f2((uint32_t)v4.x), f1 = bf16x2_to_f2((uint32_t)v4.y);
                                        const float2 f2 = bf16x2_to_f2((uint32_t)v4.z), f3 = bf16x2_to_f2((uint32_t)v4.w);
                                        outw[h2 * 2] = pack_e4m3x4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
                                        outw[h2 * 2 + 1] = pack_e4m3x4(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
                                    }
                                    q8[ci * 2 + jj] = make_int4((int)outw[0], (int)outw[1], (int)outw[2], (int)outw[3]);
                                }
                            // 64 bytes per row go out like 32 BF16 columns: whole row pieces per store instruction
                            uint8_t* obase = p.c_fp8 + (size_t)(ti.c_row + q * 32) * ldc + ti.c_col + half * 64;
                            store_block_coalesced<32>(out_stage, q8, reinterpret_cast<__nv_bfloat16*>(obase), ldc / 2, rows_valid, lane);
                            if (half == 0 && row < ti.c_row_end) {
                                const uint32_t ex = (__float_as_uint(scale) >> 23) & 0xffu;
                                *reinterpret_cast<uint32_t*>(p.c_atoms + ((size_t)(row >> 7) * (ldc / 128) + (ti.c_col >> 7)) * 512 + (row & 31) * 16 +
                                                             ((row >> 5) & 3) * 4) = ex * 0x01010101u;
                            }
                            win_phase ^= 1;
                            continue;
                        }
                    }
#pragma unroll
                    for (int ci = 0; ci < 2; ++ci) store_block_coalesced<32>(out_stage, keep[ci], wbase + half * 64 + ci * 32, ldc, rows_valid, lane);
                    win_phase ^= 1;  // kWindows == 1: the same window, next phase
                    continue;
                } else if constexpr (kSwiGLU) {
#pragma unroll 1
                    for (int c = 0; c < C::kOutCols; c += 32) {
                        uint32_t v[32], u[32];
                        tmem_ld32(taddr + c, v);
                        tmem_ld32(taddr + kBlockN / 2 + c, u);
                        tmem_ld_wait();
                        int4 regs[4];
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float o[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[j] = silu(__uint_as_float(v[i + j])) * __uint_as_float(u[i + j]);
                            regs[i / 8] = pack8_bf16(o);
                        }
                        store_block_coalesced<32>(out_stage, regs, wbase + c, ldc, rows_valid, lane);
                    }
                } else if constexpr (C::kSplitDrain) {
                    // 256-column tile, single window, two warps per lane quarter: this warp takes 128 of the columns. They go to
                    // registers raw, the window returns to the MMA issuer, then every row leaves as one 256-byte piece (to the
                    // output matrix, or with the scatter epilogue to the row its info word names).
                    uint32_t v[4][32];
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) tmem_ld32(taddr + half * 128 + c4 * 32, v[c4]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) release_window(&tmem_empty[win]);
                    int4 regs[16];
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4)
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float o[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(v[c4][i + j]);
                            regs[c4 * 4 + i / 8] = pack8_bf16(o);
                        }
                    __nv_bfloat16* dst = scatter ? (scat_ptr != nullptr ? scat_ptr + half * 128 : nullptr) : (row < ti.c_row_end ? crow + half * 128 : nullptr);
                    store_rows_256(out_stage, regs, dst, lane);
                    win_phase ^= 1;  // kWindows == 1: the same window, next phase
                    continue;
                } else if constexpr (kRowScatter) {
                    // the tile's 128 columns of every row leave as one 256-byte piece: both halves go through the staging buffer
                    // (32 rows x 16 pieces of 16 bytes, XOR-swizzled), then each store instruction covers two whole rows
                    __syncwarp();
#pragma unroll 1
                    for (int c = 0; c < 128; c += 64) {
                        uint32_t v[32], u[32];
                        tmem_ld32(taddr + c, v);
                        tmem_ld32(taddr + c + 32, u);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float o[8], o2[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                o[j] = __uint_as_float(v[i + j]);
                                o2[j] = __uint_as_float(u[i + j]);
                            }
                            out_stage[lane * 16 + ((c / 8 + i / 8) ^ (lane & 15))] = pack8_bf16(o);
                            out_stage[lane * 16 + ((c / 8 + 4 + i / 8) ^ (lane & 15))] = pack8_bf16(o2);
                        }
                    }
                    __syncwarp();
                    const unsigned long long mine = reinterpret_cast<unsigned long long>(scat_ptr);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int r2 = i * 2 + (lane >> 4), piece = lane & 15;
                        const int4 val = out_stage[r2 * 16 + (piece ^ (r2 & 15))];
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, mine, r2));
                        if (dst != nullptr) *reinterpret_cast<int4*>(dst + piece * 8) = val;
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < C::kOutCols; c += 64) {
                        uint32_t v[32], u[32];
                        tmem_ld32(taddr + c, v);
                        tmem_ld32(taddr + c + 32, u);
                        tmem_ld_wait();
                        int4 regs[8];
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float o[8], o2[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                o[j] = __uint_as_float(v[i + j]);
                                o2[j] = __uint_as_float(u[i + j]);
                            }
                            regs[i / 8] = pack8_bf16(o);
                            regs[4 + i / 8] = pack8_bf16(o2);
                        }
                        if (scatter) store_block_scattered<64>(out_stage, regs, scat_ptr != nullptr ? scat_ptr + c : nullptr, lane);
                        else store_block_coalesced<64>(out_stage, regs, wbase + c, ldc, rows_valid, lane);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) release_window(&tmem_empty[win]);
                if (++win == C::kWindows) {
                    win = 0;
                    win_phase ^= 1;
                }
            }
        }
    }

    if (warp >= 2) {
        // rows scattered into other GPUs' memory are performed there before this kernel counts as finished
        if (p.row_info != nullptr) __threadfence_system();
        if (p.trace != nullptr && warp == 2 && lane == 0) atomicMax(&p.trace[1], global_timer_ns());
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // neither CTA leaves while the other may still signal it or read its operands
    if (threadIdx.x == 0 && s_abort && p.error_flag != nullptr) atomicExch(p.error_flag, 1);
    if (warp == 1) {
        tc_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, C::kTmemCols);
        else tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---- host side ------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

// 2-D row-major [rows, cols] tensor, box = 128 bytes of columns x box_rows rows, 128B swizzle.
bool make_map(CUtensorMap* map, const void* ptr, bool fp8, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const uint64_t esz = fp8 ? 1 : 2;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * esz};
    cuuint32_t box[2] = {(cuuint32_t)(kKBlockBytes / esz), box_rows};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// 2-D row-major [k_rows, mn_cols] bf16 tensor whose contiguous dimension is the operand's row index (MN-major operand):
// box = 64 columns (128 bytes) x 64 rows, 128B swizzle.
bool make_map_mn(CUtensorMap* map, const void* ptr, uint64_t k_rows, uint64_t mn_cols) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {mn_cols, k_rows};
    cuuint64_t strides[1] = {mn_cols * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Scale atoms as a 2-D tensor of 32-bit words: one row per (tile, K block), `words` words per row (128 per 512-byte atom).
bool make_map_sf(CUtensorMap* map, const void* ptr, uint64_t rows, uint32_t words) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {words, rows};
    cuuint64_t strides[1] = {(cuuint64_t)words * 4};
    cuuint32_t box[2] = {words, 1};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int kBlockN, bool kFp8, bool kSwiGLU, bool kPair, bool kMx = false, bool kRowScatter = false>
cudaError_t launch_impl(const GroupedGemmArgs& a, cudaStream_t stream) {
    using C = Cfg<kBlockN, kFp8, kSwiGLU, kPair, kMx, kRowScatter>;
    CUtensorMap map_a, map_b, map_sfa, map_sfb;
    std::memset(&map_sfa, 0, sizeof(map_sfa));
    std::memset(&map_sfb, 0, sizeof(map_sfb));
    if constexpr (kMx && kPair) {
        const uint64_t nkb = (uint64_t)a.k / 128;
        if (!make_map_sf(&map_sfa, a.sfa_atoms, (((uint64_t)a.m_total + 127) / 128) * nkb, 128) ||
            !make_map_sf(&map_sfb, a.sfb_atoms, (uint64_t)a.num_groups * (a.n / kBlockN) * nkb, 128 * C::kSfBAtoms))
            return cudaErrorInvalidValue;
    }
    const uint32_t b_box_rows = (kSwiGLU || kPair) ? kBlockN / 2 : kBlockN;
    bool ok;
    if (a.mode == 0) {
        ok = make_map(&map_a, a.a, kFp8, (uint64_t)a.m_total, (uint64_t)a.k, kBlockM) &&
             (a.b_mn ? make_map_mn(&map_b, a.b, (uint64_t)a.num_groups * a.k, (uint64_t)a.n)  // B given as [G, K, N]
                     : make_map(&map_b, a.b, kFp8, (uint64_t)a.num_groups * a.n, (uint64_t)a.k, b_box_rows));
    } else {
        ok = (a.a_mn ? make_map_mn(&map_a, a.a, (uint64_t)a.m_total, (uint64_t)a.n)   // A given as [M, N_out]
                     : make_map(&map_a, a.a, kFp8, (uint64_t)a.n, (uint64_t)a.m_total, kBlockM)) &&
             (a.b_mn ? make_map_mn(&map_b, a.b, (uint64_t)a.m_total, (uint64_t)a.k)   // B given as [M, K_out]
                     : make_map(&map_b, a.b, kFp8, (uint64_t)a.k, (uint64_t)a.m_total, b_box_rows));
    }
    if (!ok) return cudaErrorInvalidValue;
    auto kernel = grouped_gemm_kernel<kBlockN, kFp8, kSwiGLU, kPair, kMx, kRowScatter>;
    static bool smem_opted_in[64] = {};  // per device, once: the attribute is sticky
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !smem_opted_in[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) smem_opted_in[dev] = true;
    }
    if constexpr (kPair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(a.num_sms & ~1), 1, 1);  // whole CTA pairs
        cfg.blockDim = dim3(C::kThreads, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cfg.gridDim.x < 2) return cudaErrorInvalidValue;
        return cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_sfa, map_sfb, a);
    } else {
        kernel<<<a.num_sms, C::kThreads, C::kSmemBytes, stream>>>(map_a, map_b, map_sfa, map_sfb, a);
        return cudaGetLastError();
    }
}

// kPair chosen at run time (GroupedGemmArgs::cta_pairs)
template <int kBlockN, bool kFp8, bool kSwiGLU>
cudaError_t launch_sel(const GroupedGemmArgs& a, cudaStream_t stream) {
    if (a.cta_pairs) return launch_impl<kBlockN, kFp8, kSwiGLU, true>(a, stream);
    return launch_impl<kBlockN, kFp8, kSwiGLU, false>(a, stream);
}

}  // namespace

cudaError_t launch_grouped_gemm(const GroupedGemmArgs& a, cudaStream_t stream) {
    if (a.num_groups < 1 || a.num_groups > kMaxGroups || a.num_sms < 1) return cudaErrorInvalidValue;
    // MN-major operands: bf16, no swiglu, single CTAs; mode 0 takes B that way (input gradients read the weight in place),
    // mode 1 takes both (weight gradients read the output gradient and the activation in place)
    if ((a.a_mn || a.b_mn) && (a.fp8 || a.swiglu || a.cta_pairs || (a.mode == 0 && a.a_mn) || (a.mode == 1 && !(a.a_mn && a.b_mn)) || a.n % 64 != 0))
        return cudaErrorInvalidValue;
    if (a.m_total <= 0) return cudaSuccess;
    const int kb = a.fp8 ? 128 : 64;
    if (a.mode == 0) {
        if (a.k % kb != 0) return cudaErrorInvalidValue;
        if (a.fp8 && a.sfa_atoms != nullptr) {
            // native block scaling: pre-built UE8M0 scale atoms, every group starts on a multiple of 128 rows
            if (a.sfb_atoms == nullptr || a.k % 128 != 0 || a.n % 128 != 0) return cudaErrorInvalidValue;
            if (a.swiglu) {
                if ((a.n / 2) % 128 != 0) return cudaErrorInvalidValue;  // gate/up halves start on scale-block boundaries
                if (a.mx_wide && a.cta_pairs) return launch_impl<256, true, true, true, true>(a, stream);
                if (a.mx_wide) return launch_impl<256, true, true, false, true>(a, stream);
                return launch_impl<128, true, true, false, true>(a, stream);
            }
            if (a.mx_wide) return (a.n % 256 == 0) ? launch_impl<256, true, false, false, true>(a, stream) : cudaErrorInvalidValue;
            if (a.row_info != nullptr) return launch_impl<128, true, false, false, true, true>(a, stream);
            return launch_impl<128, true, false, false, true>(a, stream);
        }
        if (a.fp8) {
            if (a.a_scales == nullptr || a.b_scales == nullptr || a.k % 128 != 0) return cudaErrorInvalidValue;
            if (a.swiglu) {
                if ((a.n / 2) % 128 != 0) return cudaErrorInvalidValue;  // gate/up halves must start on scale-block boundaries
                return launch_sel<128, true, true>(a, stream);
            }
            if (a.n % 128 != 0) return cudaErrorInvalidValue;
            return launch_sel<128, true, false>(a, stream);
        }
        if (a.swiglu) {
            if ((a.n / 2) % 128 == 0) return launch_sel<256, false, true>(a, stream);
            if ((a.n / 2) % 64 == 0) return launch_sel<128, false, true>(a, stream);
            return cudaErrorInvalidValue;
        }
        if (a.n % 256 == 0) return launch_sel<256, false, false>(a, stream);
        if (a.n % 128 == 0) return launch_sel<128, false, false>(a, stream);
        return cudaErrorInvalidValue;
    }
    // K-grouped (weight gradients), bf16 only
    if (a.fp8 || a.swiglu || a.n % kBlockM != 0) return cudaErrorInvalidValue;
    if (a.k % 256 == 0) return launch_sel<256, false, false>(a, stream);
    if (a.k % 128 == 0) return launch_sel<128, false, false>(a, stream);
    return cudaErrorInvalidValue;
}

}  // namespace dx
