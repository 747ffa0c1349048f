// Batched dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
//   Y[m, n] = sum_k X[m, k] * W[n, k],  W quantized (any supported format), X/Y f32.
//
// The reference has no batched GPU path at all (its GPU prefill is token-by-token GEMV,
// src/main.rs:1410-1416); its CPU form is dequant::gemm (src/dequant.rs:143-200).
//
// Persistent kernel, one CTA per SM (two for narrow token tiles).  Every CTA first takes as many whole
// tiles as all CTAs can get; the (row tile, token tile, K step) units of the remaining tiles, tile-major,
// are cut into one equal contiguous share per CTA.  A tile is
// 128 or 256 weight rows (one or two UMMA M=128 accumulators side by side in TMEM) x up to 256 tokens
// (the UMMA N dimension).  Per 64-wide K step of a tile:
//   * producer warps -- two groups that take alternate K steps, one thread per weight row --
//     dequantize the weight tile to bf16 straight into shared memory in the K-major 128-byte-swizzled
//     layout tcgen05.mma reads (raw bytes of the thread's next step are loaded into registers while the
//     current one is unpacked; Q4_K / Q6_K use packed bf16x2 arithmetic: nibble|0x4300 is the bf16
//     128+q, an exact HSUB2 removes the 128, one HFMA2 applies scale and min; IQ2_XS / IQ3_XXS read
//     bf16 grids and sign bytes from shared-memory tables), and one thread starts the bulk async copy
//     of the step's pre-swizzled bf16 activation tile;
//   * they fence the generic->async proxy and arrive on the stage's "full" mbarrier;
//   * one elected thread issues four tcgen05.mma per accumulator (K=16 each, kind::f16, bf16 x bf16 ->
//     f32 in TMEM) and a tcgen05.commit that arrives on the stage's "empty" mbarrier when the tensor
//     core has finished reading the stage.
// A 3-4 stage ring lets dequantization run ahead of the MMAs.  Dedicated epilogue warps read a finished
// tile's accumulator with tcgen05.ld (32 lanes x 32 columns per instruction), one weight row per thread,
// and store it -- or, for a tile that two CTAs share, add it atomically onto zeros -- into the
// token-major output, then hand the accumulator back to the MMA thread.
//
// Within every group of four consecutive k the tile order is (0,2,1,3) for BOTH operands: that
// is the order byte->bf16x2 unpacking produces for free, and a contraction does not care about
// a permutation applied to both sides.  The activation tile is converted f32->bf16 (and
// permuted) once per call by convert_x_bf16_kernel.
//
// Every mbarrier wait is bounded (~1 s); a timeout sets the status word, the loops are left,
// and the CTA still reaches the common exit where the allocating warp frees its TMEM columns.
#pragma once

#include <cuda_bf16.h>

#include "formats.cuh"
#include "gemv_tma.cuh"

namespace qz {

constexpr int GEMM_ROWS = 128;       // UMMA M
constexpr int GEMM_KSTEP = 64;       // one 128-byte swizzle atom of bf16
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_MAX_TOKENS = 256; // UMMA N per CTA

// A grouped problem (mixture-of-experts): the rows of the activation matrix are slots grouped by expert,
// slot ranges and tile counts live in DEVICE memory (built by moe_route_kernel), so the host never needs to
// know them.  One launch then runs, for every expert e and each of n_mats stacked weight tensors,
//   Ym[mat][slot, :] = Xtiles(e) * Wm[mat][e]^T     for the slots of expert e.
constexpr int QZ_MOE_MAX_E = 256;
struct GemmGroup {
    int n_experts;
    int n_tt_total;                      // token tiles of all experts together
    int counts[QZ_MOE_MAX_E];            // slots of expert e
    int offsets[QZ_MOE_MAX_E + 1];       // first slot of expert e
    int tt_prefix[QZ_MOE_MAX_E + 1];     // token tiles before expert e (a token tile = tok_tile slots of one expert)
};

struct GemmArgs {
    const GemmGroup *grp;      // NULL: one plain GEMM (W, Y, M below)
    const uint8_t *Wm[2];      // grouped: stacked expert tensors, expert e at + e * expert_stride
    float *Ym[2];              // grouped: outputs [slots, N]
    size_t expert_stride;
    int n_mats;
    const uint8_t *W;
    const __nv_bfloat16 *Xb;   // bf16 activation tiles, pre-swizzled (see convert_x_bf16_kernel)
    float *Y;                  // [M, N] token-major
    int M, K, N;
    int planes;                // weight layout
    int n_tok_tiles, tok_tile; // tokens per CTA (multiple of 16, <= 256)
    long long units;           // (tile, K step) units in all, tile-major
    long long dp_units;        // whole-tile part: CTA c owns units [c * dp_units, (c + 1) * dp_units)
    long long rem_begin;       // first unit of the shared part (= CTAs x dp_units)
    long long units_per_cta;   // shared part: CTA c owns [rem_begin + c * units_per_cta, + units_per_cta), clipped
    int stages;                // MMA ring depth
    int *status;
    // row-sharded GEMM (push.n > 0): the epilogue stores every output element into ALL ranks' windows, token m /
    // local row n at push_off + m * push_ld + n, straight from the accumulator, and the last CTA publishes the
    // exchange.  The host uses this form only with a schedule of whole tiles (no tile shared between CTAs).
    PushArgs push;
    long long push_off, push_ld;
};

// ---- f32 or bf16 [M,K] -> bf16 tiles in exactly the shared-memory image the MMA reads: for every
//      (token tile, K step) a contiguous [tok_tile rows x 128 B] block, 16-byte chunk c of row r stored
//      at chunk c ^ (r & 7), k order (0,2,1,3) inside every four.  A stage's activation tile is then
//      ONE bulk async copy.  One thread per 16-byte chunk.
//      perm = 1 (Q6_K weight tiles): position p of K step (block b, j) holds activation
//      256 b + 128 (j >> 1) + 32 (p >> 4) + 16 (j & 1) + (p & 15): the K order in which the Q6_K producer
//      emits weights (all four 32-runs of one 16-wide slice, so that every loaded bit is used). ----
template <bool IN_BF16>
__global__ void convert_x_bf16_kernel(const void *__restrict__ xin, __nv_bfloat16 *__restrict__ out, int M, int K,
                                      int tok_tile, int n_tok_tiles, int perm)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int ksteps = K / 64;
    const long long total = (long long)n_tok_tiles * tok_tile * ksteps * 8;
    if (i >= total) return;
    const int c = (int)(i & 7);
    long long rest = i >> 3;
    const int r = (int)(rest % tok_tile);
    rest /= tok_tile;
    const int ks = (int)(rest % ksteps);
    const int tile = (int)(rest / ksteps);
    const int tok = tile * tok_tile + r;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (tok < M) {
        const int p = 8 * c;   // first of this chunk's eight tile positions: they stay contiguous in x
        const int koff = perm ? 256 * (ks >> 2) + 128 * ((ks >> 1) & 1) + 32 * (p >> 4) + 16 * (ks & 1) + (p & 15) : ks * 64 + p;
        if (IN_BF16) {
            // eight bf16 values e0..e7 -> words (e0,e2) (e1,e3) (e4,e6) (e5,e7)
            const uint4 v = *(const uint4 *)((const uint16_t *)xin + (size_t)tok * K + koff);
            o = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632), __byte_perm(v.z, v.w, 0x5410),
                           __byte_perm(v.z, v.w, 0x7632));
        } else {
            const float *src = (const float *)xin + (size_t)tok * K + koff;
            const float4 v0 = *(const float4 *)src, v1 = *(const float4 *)(src + 4);
            __nv_bfloat162 a = __floats2bfloat162_rn(v0.x, v0.z), b = __floats2bfloat162_rn(v0.y, v0.w);
            __nv_bfloat162 d = __floats2bfloat162_rn(v1.x, v1.z), e = __floats2bfloat162_rn(v1.y, v1.w);
            o = make_uint4(*(uint32_t *)&a, *(uint32_t *)&b, *(uint32_t *)&d, *(uint32_t *)&e);
        }
    }
    uint8_t *tile_base = (uint8_t *)out + ((size_t)tile * ksteps + ks) * ((size_t)tok_tile * 128);
    *(uint4 *)(tile_base + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = o;
}

// ---- tcgen05 / TMEM primitives ----
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 16 / 32 consecutive columns per instruction: one round trip to tensor memory per 16 / 32
// tokens instead of one per 8 (the round trip, not the data volume, is what an epilogue waits for)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Bounded mbarrier wait that sleeps between polls: the waiting warps (producers ahead of the tensor
// core, epilogue warps idle for a whole tile) leave the issue slots to the warps that unpack.
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t *bar, uint32_t parity, unsigned ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    do {
        __nanosleep(ns);
        if (mbar_try_wait(bar, parity)) return true;
    } while (clock64() - t0 <= TMA_WAIT_CYCLES);
    return false;
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);    // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                        // layout type: SWIZZLE_128B
    return d;
}
// Instruction descriptor: D = f32, A = B = bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(GEMM_ROWS >> 4) << 24);
}

// position of 16-byte chunk c of row r inside a [rows x 128 B] swizzled tile
__device__ __forceinline__ uint32_t sw128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// four bytes (values < 128) -> two bf16x2 registers holding (b0, b2) and (b1, b3) minus `bias`,
// times `scale`, minus `sub` (all packed bf16x2 constants)
__device__ __forceinline__ void bytes4_to_bf16(uint32_t v, __nv_bfloat162 bias, __nv_bfloat162 scale, __nv_bfloat162 sub,
                                               uint32_t &o02, uint32_t &o13)
{
    uint32_t t02 = (v & 0x00FF00FFu) | 0x43004300u, t13 = ((v >> 8) & 0x00FF00FFu) | 0x43004300u;
    __nv_bfloat162 a = __hsub2(*(__nv_bfloat162 *)&t02, bias), b = __hsub2(*(__nv_bfloat162 *)&t13, bias);
    a = __hfma2(a, scale, sub);
    b = __hfma2(b, scale, sub);
    o02 = *(uint32_t *)&a;
    o13 = *(uint32_t *)&b;
}

// L2 prefetch of a row's bytes a few blocks ahead of the loads: one thread walks one weight row, 16 to 48 bytes per
// K step, so without it every load is a full HBM round trip and only a few KB per SM are ever in flight (the
// kernel then runs at a few percent of the DRAM bandwidth, bound by that latency).  `pf` 256-weight blocks ahead
// (GEMM_PF_BLOCKS, or 0 = off), issued once per block by the thread that handles the block's first K step; never
// past the row's end.
#ifndef QZ_GEMM_PF_BLOCKS
#define QZ_GEMM_PF_BLOCKS 2
#endif
constexpr int GEMM_PF_BLOCKS = QZ_GEMM_PF_BLOCKS;
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ---- A-tile producers: one thread per weight row and K step (64 weights = the tile row's eight
//      16-byte chunks).  load() only issues the global loads of a K step into registers, so they
//      are in flight while the thread's previous step is unpacked; store() unpacks to bf16 and
//      writes the swizzled tile row. ----
template <uint32_t T, bool PLANES>
struct AProd {   // generic: any format, either layout, through the bit-exact decoder; no prefetch
    struct Raw { int unused; };
    static constexpr bool TWO_SETS = false;
    static constexpr int TABLE_BYTES = 0;
    __device__ static void build_table(uint8_t *, int, int) {}
    __device__ static void load(Raw &, const uint8_t *, int, int, int) {}
    __device__ static void store(uint8_t *As, const Raw &, const uint8_t *rowp, int nb, int kstep, int r, const uint8_t *)
    {
        const FormatInfo fi = format_info(T);
#pragma unroll 1
        for (int h = 0; h < 2; h++) {
            const int elem0 = kstep * GEMM_KSTEP + 32 * h;
            float w[32];
            if (rowp) {
                Fields F = block_fields<PLANES>(fi, rowp, nb, elem0 / fi.block_elems);
                decode32<T>(F, (elem0 % fi.block_elems) / 32, w);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) w[i] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    __nv_bfloat162 a = __floats2bfloat162_rn(w[8 * c + 4 * j], w[8 * c + 4 * j + 2]);
                    __nv_bfloat162 b = __floats2bfloat162_rn(w[8 * c + 4 * j + 1], w[8 * c + 4 * j + 3]);
                    o[2 * j] = *(uint32_t *)&a;
                    o[2 * j + 1] = *(uint32_t *)&b;
                }
                *(uint4 *)(As + sw128(r, 4 * h + c)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
};

// Q4_K, raw layout: K step = sub-block pair p of block b (low nibbles: sub-block 2p, high: 2p+1)
template <>
struct AProd<T_Q4_K, false> {
    struct Raw { uint4 hdr, q0, q1; };
    static constexpr bool TWO_SETS = true;
    static constexpr int TABLE_BYTES = 0;
    __device__ static void build_table(uint8_t *, int, int) {}
    __device__ static void load(Raw &w, const uint8_t *rowp, int nb, int kstep, int pf)
    {
        if (rowp) {
            const uint8_t *blk = rowp + (size_t)(kstep >> 2) * 144;
            const int p = kstep & 3;
            // (144-byte blocks: the line that holds a block's last byte is the one no earlier block has asked for)
            if (pf > 0 && p == 0 && (kstep >> 2) + pf < nb) prefetch_l2(blk + pf * 144 + 143);
            w.hdr = __ldg((const uint4 *)blk);
            w.q0 = __ldg((const uint4 *)(blk + 16 + 32 * p));
            w.q1 = __ldg((const uint4 *)(blk + 32 + 32 * p));
        } else {
            w.hdr = w.q0 = w.q1 = make_uint4(0, 0, 0, 0);
        }
    }
    __device__ static void store(uint8_t *As, const Raw &w, const uint8_t *, int, int kstep, int r, const uint8_t *)
    {
        const uint32_t q[8] = {w.q0.x, w.q0.y, w.q0.z, w.q0.w, w.q1.x, w.q1.y, w.q1.z, w.q1.w};
        const int p = kstep & 3;
        // the 12 packed 6-bit codes (src/dequant.rs:1471-1480), as three words
        const uint32_t s0 = w.hdr.y, s1 = w.hdr.z, s2 = w.hdr.w;
        const uint32_t scw = p < 2 ? (s0 & 0x3F3F3F3Fu) : ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u));
        const uint32_t mw = p < 2 ? (s1 & 0x3F3F3F3Fu) : (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u));
        const int sh = 16 * (p & 1);
        const float2 dm = __half22float2(*(const __half2 *)&w.hdr.x);
        const __nv_bfloat162 bias = __floats2bfloat162_rn(128.f, 128.f);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float d1 = dm.x * (float)((scw >> (sh + 8 * h)) & 0xFF), m1 = dm.y * (float)((mw >> (sh + 8 * h)) & 0xFF);
            const __nv_bfloat162 scale = __floats2bfloat162_rn(d1, d1), sub = __floats2bfloat162_rn(-m1, -m1);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[4];
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    const uint32_t v = (h ? (q[2 * c + jj] >> 4) : q[2 * c + jj]) & 0x0F0F0F0Fu;
                    bytes4_to_bf16(v, bias, scale, sub, o[2 * jj], o[2 * jj + 1]);
                }
                *(uint4 *)(As + sw128(r, 4 * h + c)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
};

// Q6_K, plane layout (ql[nb x 128] | qh[nb x 64] | scales[nb x 16] | d[nb x 2]): weight 128 n + 32 k + l of
// a block takes the nibble (k >> 1) of ql[64 n + 32 (k & 1) + l], bits 2k, 2k+1 of qh[32 n + l] and scale
// 8 n + 2 k + l / 16 (src/dequant.rs:1583-1631).  K step j of a block = half n = j >> 1, slice
// l in [16 (j & 1), +16), ALL four runs k: 16 + 16 bytes of ql (both nibbles used), 16 bytes of qh (all four
// bit pairs used), one scale per run.  Tile position p = 16 k + (l & 15); the activation tiles are built
// in the same order (convert_x_bf16_kernel, perm = 1).
template <>
struct AProd<T_Q6_K, true> {
    struct Raw { uint4 a0, a1, h; uint2 sc; uint32_t d; };
    static constexpr bool TWO_SETS = true;
    static constexpr int TABLE_BYTES = 0;
    __device__ static void build_table(uint8_t *, int, int) {}
    __device__ static void load(Raw &w, const uint8_t *rowp, int nb, int kstep, int pf)
    {
        if (rowp) {
            const int b = kstep >> 2, n = (kstep >> 1) & 1, lh = kstep & 1;
            if (pf > 0 && (kstep & 3) == 0 && b + pf < nb) {   // ql: one line per block; qh: one line per two blocks
                prefetch_l2(rowp + (size_t)(b + pf) * 128);
                if ((b & 1) == 0) prefetch_l2(rowp + (size_t)nb * 128 + (size_t)(b + pf) * 64);
                if ((b & 7) == 0) prefetch_l2(rowp + (size_t)nb * 192 + (size_t)(b + pf) * 16);
            }
            const uint8_t *pl = rowp + (size_t)b * 128 + 64 * n + 16 * lh;
            w.a0 = __ldg((const uint4 *)pl);            // runs 0 (low nibbles) and 2 (high nibbles)
            w.a1 = __ldg((const uint4 *)(pl + 32));     // runs 1 and 3
            w.h = __ldg((const uint4 *)(rowp + (size_t)nb * 128 + (size_t)b * 64 + 32 * n + 16 * lh));
            w.sc = __ldg((const uint2 *)(rowp + (size_t)nb * 192 + (size_t)b * 16 + 8 * n));
            w.d = __ldg((const uint16_t *)(rowp + (size_t)nb * 208 + (size_t)b * 2));
        } else {
            w.a0 = w.a1 = w.h = make_uint4(0, 0, 0, 0);
            w.sc = make_uint2(0, 0);
            w.d = 0;
        }
    }
    __device__ static void store(uint8_t *As, const Raw &w, const uint8_t *, int, int kstep, int r, const uint8_t *)
    {
        const uint32_t ql[2][4] = {{w.a0.x, w.a0.y, w.a0.z, w.a0.w}, {w.a1.x, w.a1.y, w.a1.z, w.a1.w}};
        const uint32_t qh[4] = {w.h.x, w.h.y, w.h.z, w.h.w};
        const int lh = kstep & 1;
        const float d = h2f((uint16_t)w.d);
        const __nv_bfloat162 bias = __floats2bfloat162_rn(160.f, 160.f);   // the bf16 magic 128 plus Q6_K's own 32
        const __nv_bfloat162 zero = __floats2bfloat162_rn(0.f, 0.f);
        // scale bytes 2k + lh, k = 0..3, of the half's eight
        const uint32_t s4 = lh ? __byte_perm(w.sc.x, w.sc.y, 0x7531) : __byte_perm(w.sc.x, w.sc.y, 0x6420);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float sk = d * (float)(int8_t)((s4 >> (8 * k)) & 0xFF);
            const __nv_bfloat162 sc = __floats2bfloat162_rn(sk, sk);
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t v = ((ql[k & 1][i] >> (4 * (k >> 1))) & 0x0F0F0F0Fu) | (((qh[i] >> (2 * k)) & 0x03030303u) << 4);
                bytes4_to_bf16(v, bias, sc, zero, o[2 * i], o[2 * i + 1]);
            }
            *(uint4 *)(As + sw128(r, 2 * k)) = make_uint4(o[0], o[1], o[2], o[3]);
            *(uint4 *)(As + sw128(r, 2 * k + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
};

// ---- codebook formats: the grids are kept in shared memory already converted to bf16 and already in
//      tile order ((w0,w2),(w1,w3) per four weights), next to the 128 sign bytes.  Eight weights then cost
//      one or two grid reads, one byte read, the mask arithmetic, four XORs and four HMUL2s. ----
__device__ __forceinline__ uint32_t bf16x2_of(float a, float b)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *(uint32_t *)&v;
}
// The sign bytes (one bit per weight of a group of eight) are kept in shared memory as they are: 128 bytes, one
// row of banks, so a warp's 32 random reads never conflict.  sign_masks() spreads a byte into the XOR masks of the
// eight bf16 weights in tile order, words (s0,s2) (s1,s3) (s4,s6) (s5,s7): a dozen integer instructions instead
// of a 16-byte table entry per group (random 16-byte reads conflict two- to three-fold).
__device__ __forceinline__ void build_sign_table(uint8_t *dst, int tid, int n)
{
    for (int i = tid; i < 128; i += n) dst[i] = g_ksigns[i];
}
__device__ __forceinline__ uint4 sign_masks(uint32_t s)
{
    return make_uint4(((s & 1u) << 15) | ((s & 4u) << 29), ((s & 2u) << 14) | ((s & 8u) << 28),
                      ((s & 16u) << 11) | ((s & 64u) << 25), ((s & 32u) << 10) | ((s & 128u) << 24));
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, __nv_bfloat162 s)
{
    __nv_bfloat162 r = __hmul2(*(__nv_bfloat162 *)&a, s);
    return *(uint32_t *)&r;
}

// IQ2_XS, plane layout (d[nb x 2] | qs[nb x 64] | scales[nb x 8]): K step = the 64 weights of pair p
// of block b: eight u16 (9-bit grid index, 7-bit sign index), two scale bytes (src/dequant.rs:1043-1075)
template <>
struct AProd<T_IQ2_XS, true> {
    struct Raw { uint4 q; uint32_t sc, d; };
    static constexpr bool TWO_SETS = true;
    static constexpr int TABLE_BYTES = 512 * 16 + 128;
    __device__ static void build_table(uint8_t *tbl, int tid, int n)
    {
        uint4 *g = (uint4 *)tbl;
        for (int i = tid; i < 512; i += n) {
            const uint64_t v = g_iq2xs_grid[i];
            auto b = [&](int j) { return (float)(int)(int8_t)(v >> (8 * j)); };
            g[i] = make_uint4(bf16x2_of(b(0), b(2)), bf16x2_of(b(1), b(3)), bf16x2_of(b(4), b(6)), bf16x2_of(b(5), b(7)));
        }
        build_sign_table((uint8_t *)(g + 512), tid, n);
    }
    __device__ static void load(Raw &w, const uint8_t *rowp, int nb, int kstep, int pf)
    {
        if (rowp) {
            const int b = kstep >> 2, p = kstep & 3;
            if (pf > 0 && p == 0 && (b & 1) == 0 && b + pf < nb)   // qs: one 128-byte line per two blocks
                prefetch_l2(rowp + (size_t)nb * 2 + (size_t)(b + pf) * 64);
            w.q = __ldg((const uint4 *)(rowp + (size_t)nb * 2 + (size_t)b * 64 + 16 * p));
            w.sc = __ldg((const uint16_t *)(rowp + (size_t)nb * 66 + (size_t)b * 8 + 2 * p));
            w.d = __ldg((const uint16_t *)(rowp + (size_t)b * 2));
        } else {
            w.q = make_uint4(0, 0, 0, 0);
            w.sc = w.d = 0;
        }
    }
    __device__ static void store(uint8_t *As, const Raw &w, const uint8_t *, int, int, int r, const uint8_t *tbl)
    {
        const uint4 *grid = (const uint4 *)tbl;
        const uint8_t *sign = (const uint8_t *)(grid + 512);
        const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        const float d = 0.25f * h2f((uint16_t)w.d);
#pragma unroll
        for (int l = 0; l < 8; l++) {
            const uint32_t q = (qw[l >> 1] >> (16 * (l & 1))) & 0xFFFF;
            const uint32_t nib = (w.sc >> (8 * (l >> 2) + 4 * ((l >> 1) & 1))) & 0xF;
            const float db = d * (0.5f + (float)nib);
            const __nv_bfloat162 s2 = __floats2bfloat162_rn(db, db);
            const uint4 g = grid[q & 511], m = sign_masks(sign[q >> 9]);
            *(uint4 *)(As + sw128(r, l)) = make_uint4(hmul2_bits(g.x ^ m.x, s2), hmul2_bits(g.y ^ m.y, s2),
                                                      hmul2_bits(g.z ^ m.z, s2), hmul2_bits(g.w ^ m.w, s2));
        }
    }
};

// IQ3_XXS, plane layout (d[nb x 2] | qs[nb x 64] | scales_and_signs[nb x 32]): K step = pair p of block b:
// sixteen grid-index bytes (four weights each) and two u32 (4 x 7 sign bits + 4-bit scale per 32 weights)
template <>
struct AProd<T_IQ3_XXS, true> {
    struct Raw { uint4 q; uint2 sas; uint32_t d; };
    static constexpr bool TWO_SETS = true;
    static constexpr int TABLE_BYTES = 256 * 8 + 128;
    __device__ static void build_table(uint8_t *tbl, int tid, int n)
    {
        uint2 *g = (uint2 *)tbl;
        for (int i = tid; i < 256; i += n) {
            const uint32_t v = g_iq3xxs_grid[i];
            auto b = [&](int j) { return (float)((v >> (8 * j)) & 0xFF); };
            g[i] = make_uint2(bf16x2_of(b(0), b(2)), bf16x2_of(b(1), b(3)));
        }
        build_sign_table(tbl + 256 * 8, tid, n);
    }
    __device__ static void load(Raw &w, const uint8_t *rowp, int nb, int kstep, int pf)
    {
        if (rowp) {
            const int b = kstep >> 2, p = kstep & 3;
            if (pf > 0 && p == 0 && (b & 1) == 0 && b + pf < nb) {   // qs: a line per two blocks; signs/scales: per four
                prefetch_l2(rowp + (size_t)nb * 2 + (size_t)(b + pf) * 64);
                if ((b & 3) == 0) prefetch_l2(rowp + (size_t)nb * 66 + (size_t)(b + pf) * 32);
            }
            w.q = __ldg((const uint4 *)(rowp + (size_t)nb * 2 + (size_t)b * 64 + 16 * p));
            w.sas = __ldg((const uint2 *)(rowp + (size_t)nb * 66 + (size_t)b * 32 + 8 * p));
            w.d = __ldg((const uint16_t *)(rowp + (size_t)b * 2));
        } else {
            w.q = make_uint4(0, 0, 0, 0);
            w.sas = make_uint2(0, 0);
            w.d = 0;
        }
    }
    __device__ static void store(uint8_t *As, const Raw &w, const uint8_t *, int, int, int r, const uint8_t *tbl)
    {
        const uint2 *grid = (const uint2 *)tbl;
        const uint8_t *sign = tbl + 256 * 8;
        const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        const float d = 0.5f * h2f((uint16_t)w.d);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a1 = h ? w.sas.y : w.sas.x;
            const float db = d * (0.5f + (float)(a1 >> 28));
            const __nv_bfloat162 s2 = __floats2bfloat162_rn(db, db);
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t two = (qw[2 * h + (l >> 1)] >> (16 * (l & 1))) & 0xFFFF;   // index bytes 2l, 2l+1
                const uint2 g1 = grid[two & 0xFF], g2 = grid[two >> 8];
                const uint4 m = sign_masks(sign[(a1 >> (7 * l)) & 127]);
                *(uint4 *)(As + sw128(r, 4 * h + l)) = make_uint4(hmul2_bits(g1.x ^ m.x, s2), hmul2_bits(g1.y ^ m.y, s2),
                                                                  hmul2_bits(g2.x ^ m.z, s2), hmul2_bits(g2.y ^ m.w, s2));
            }
        }
    }
};

template <uint32_t T, bool PLANES>
constexpr bool gemm_fast_type() { return (T == T_Q4_K && !PLANES) || (PLANES && (T == T_Q6_K || T == T_IQ2_XS || T == T_IQ3_XXS)); }

template <int HALVES>
constexpr int gemm_threads() { return 2 * 128 * HALVES + 32 + 128 * HALVES; }   // producers, MMA warp, epilogue warps

// ---- zero the output tiles that more than one CTA contributes to (their partial sums are added
//      atomically).  blockIdx.x = CTA of the GEMM grid: the first CTA whose share of the shared part begins
//      strictly inside a tile's K range zeroes that tile; blockIdx.y = slice of the tile's tokens. ----
__global__ void gemm_zero_split_tiles_kernel(float *__restrict__ Y, int M, int N, int ksteps, int n_tok_tiles, int tok_tile,
                                             int cta_rows, long long units, long long rem_begin, long long units_per_cta)
{
    const long long u0 = rem_begin + (long long)blockIdx.x * units_per_cta;
    if (u0 >= units) return;
    const long long off = u0 % ksteps;
    if (off == 0 || off > units_per_cta) return;   // not inside a tile, or not the first share to begin inside it
    const int tile = (int)(u0 / ksteps);
    const int row0 = (tile / n_tok_tiles) * cta_rows, tok0 = (tile % n_tok_tiles) * tok_tile;
    const int rows = min(cta_rows, N - row0), toks = min(tok_tile, M - tok0);
    const int per = (toks + gridDim.y - 1) / gridDim.y;
    const int t0 = blockIdx.y * per, t1 = min(t0 + per, toks);
    if (((N | rows) & 3) == 0) {   // row0 is a multiple of 128: 16-byte stores
        const int r4 = rows >> 2;
        for (int i = threadIdx.x; i < (t1 - t0) * r4; i += blockDim.x) {
            const int tk = t0 + i / r4, rr = i - (i / r4) * r4;
            *(float4 *)(Y + (size_t)(tok0 + tk) * N + row0 + 4 * rr) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else {
        for (int i = threadIdx.x; i < (t1 - t0) * rows; i += blockDim.x) {
            const int tk = t0 + i / rows, rr = i - (i / rows) * rows;
            Y[(size_t)(tok0 + tk) * N + row0 + rr] = 0.f;
        }
    }
}

// A CTA's work: first its whole tiles (units u1 .. u1 + n1), then its share of the shared part (from u2),
// n units in all.  A cursor walks it forwards; it divides only when it is placed and when it crosses from
// the first range into the second.
struct GemmShare {
    long long u1, u2;
    int n1, n;
    int ksteps;
    struct Cursor { int i, tile, ks; };
    __device__ void place(Cursor &c, int i) const
    {
        const long long u = i < n1 ? u1 + i : u2 + (i - n1);
        c.i = i;
        c.tile = (int)(u / ksteps);
        c.ks = (int)(u - (long long)c.tile * ksteps);
    }
    __device__ void advance(Cursor &c, int by) const
    {
        if (c.i < n1 && c.i + by >= n1) {
            place(c, c.i + by);
            return;
        }
        c.i += by;
        c.ks += by;
        while (c.ks >= ksteps) {
            c.ks -= ksteps;
            c.tile++;
        }
    }
    // units from the cursor to the end of its tile or of its range, whichever comes first
    __device__ int run(const Cursor &c) const { return min(ksteps - c.ks, (c.i < n1 ? n1 : n) - c.i); }
};

// What a tile index means.  Plain GEMM: tile = row_tile * n_tok_tiles + token tile.  Grouped: tiles are
// numbered expert by expert, inside an expert matrix by matrix, inside a matrix row tile by row tile.
struct GemmTile {
    int row_tile;        // weight rows [row_tile * CTA_ROWS, +CTA_ROWS)
    int ntok;            // tokens of this tile (multiple of 16): the UMMA N
    int valid;           // tokens of this tile that exist (the rest is padding)
    size_t x_tile;       // index of the activation token tile (its K steps follow one another)
    const uint8_t *W;    // weight matrix of this tile
    float *Y;            // output row of the tile's first token
    int tok0;            // index of the tile's first token (plain GEMM)
};

struct GemmGroupView {   // the group descriptor as one CTA sees it (shared memory)
    int n_experts, n_row_tiles, n_mats;
    int tile_prefix[QZ_MOE_MAX_E + 1];   // GEMM tiles before expert e
};

__device__ __forceinline__ int group_find(const int *prefix, int n, int v)   // largest e with prefix[e] <= v
{
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= v) lo = mid;
        else hi = mid;
    }
    return lo;
}

// ---- the kernel.  Persistent.  The tiles of the whole problem, in tile-major unit order, are split in
//      two parts: as many whole tiles per CTA as every CTA can get (stored with plain stores, no other CTA
//      touches them), and the rest -- less than one tile per CTA -- whose (tile, K step) units are cut
//      into one contiguous, equally long range per CTA, so every SM gets the same amount of work whatever
//      the tile count; such a range may end inside a tile and the next CTA continues it.  A tile of the
//      second part that a single CTA covers completely is stored; a shared one is added atomically onto
//      zeros.  A CTA owns HALVES x 128 weight rows of a tile (one UMMA M=128 accumulator per half,
//      side by side in TMEM), so an activation tile fetched from L2 feeds HALVES x 128 rows.
//      Warps: 8 x HALVES producers | 1 MMA issuer + TMEM owner | 4 x HALVES epilogue. ----
template <uint32_t T, bool PLANES, int HALVES>
__global__ void __launch_bounds__(gemm_threads<HALVES>(), (gemm_fast_type<T, PLANES>() && HALVES == 1) ? 2 : 1)
    gemm_tc_kernel(const GemmArgs a)
{
    extern __shared__ __align__(1024) uint8_t gsm[];
    __shared__ uint64_t full_bar[GEMM_STAGES], empty_bar[GEMM_STAGES], done_bar, acc_free_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    using P = AProd<T, PLANES>;
    constexpr int PRODUCERS = 256 * HALVES, PWARPS = PRODUCERS / 32, CTA_ROWS = GEMM_ROWS * HALVES;

    __shared__ GemmGroupView gv;
    __shared__ long long sched[4];   // dp_units, rem_begin, units_per_cta, units

    const FormatInfo fi = format_info(T);
    const int nb = a.K / fi.block_elems;
    const size_t row_bytes = (size_t)nb * fi.block_bytes;
    const int ntok_max = a.tok_tile;                          // widest UMMA N of this launch (multiple of 16)
    const int ksteps = a.K / GEMM_KSTEP;
    const int a_bytes = CTA_ROWS * 128, b_stride = ntok_max * 128;
    const int stage_bytes = a_bytes + ((b_stride + 1023) & ~1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int acc_cols = HALVES * ntok_max;
    const uint32_t tmem_cols = acc_cols <= 32 ? 32 : (acc_cols <= 64 ? 64 : (acc_cols <= 128 ? 128 : (acc_cols <= 256 ? 256 : 512)));
    const GemmGroup *grp = a.grp;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_STAGES; s++) {
            mbar_init(&full_bar[s], PWARPS / 2 + 1);   // one group's producer warps + the activation copy
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&done_bar, 1);
        mbar_init(&acc_free_bar, 4 * HALVES);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (grp) {
            // Grouped: the tile count comes from the device-side expert counts, so every CTA derives the same
            // two-part split here that the host computes for a plain GEMM.
            const int ne = grp->n_experts;
            gv.n_experts = ne;
            gv.n_row_tiles = (a.N + CTA_ROWS - 1) / CTA_ROWS;
            gv.n_mats = a.n_mats;
            int acc = 0;
            for (int e = 0; e < ne; e++) {
                gv.tile_prefix[e] = acc;
                acc += a.n_mats * gv.n_row_tiles * ((grp->counts[e] + ntok_max - 1) / ntok_max);
            }
            gv.tile_prefix[ne] = acc;
            const long long tiles = acc, units = tiles * ksteps, ctas = gridDim.x;
            const long long whole = tiles / ctas;
            const long long dp = whole * ksteps, rem_begin = ctas * dp, rem = units - rem_begin;
            long long sharers = ctas;
            if (sharers > (rem + 7) / 8) sharers = (rem + 7) / 8;
            sched[0] = dp;
            sched[1] = rem_begin;
            sched[2] = sharers > 0 ? (rem + sharers - 1) / sharers : 0;
            sched[3] = units;
        } else {
            sched[0] = a.dp_units;
            sched[1] = a.rem_begin;
            sched[2] = a.units_per_cta;
            sched[3] = a.units;
        }
    }
    if (warp == PWARPS) tmem_alloc(&tmem_base_s, tmem_cols);   // one full warp allocates
    uint8_t *tbl = gsm + (size_t)a.stages * stage_bytes;        // codebook tables of the format, behind the ring
    P::build_table(tbl, threadIdx.x, blockDim.x);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    GemmShare sh;
    sh.ksteps = ksteps;
    sh.u1 = (long long)blockIdx.x * sched[0];
    sh.n1 = (int)sched[0];
    sh.u2 = sched[1] + (long long)blockIdx.x * sched[2];
    {
        const long long e2 = min(sh.u2 + sched[2], sched[3]);
        sh.n = sh.n1 + (e2 > sh.u2 ? (int)(e2 - sh.u2) : 0);
    }
    const int nunits = sh.n;
    auto resolve = [&](int tile) -> GemmTile {
        GemmTile t;
        if (!grp) {
            const int tt = tile % a.n_tok_tiles;
            t.row_tile = tile / a.n_tok_tiles;
            t.ntok = ntok_max;
            t.valid = min(ntok_max, a.M - tt * ntok_max);
            t.x_tile = (size_t)tt;
            t.W = a.W;
            t.Y = a.Y + (size_t)tt * ntok_max * a.N;
            t.tok0 = tt * ntok_max;
        } else {
            const int e = group_find(gv.tile_prefix, gv.n_experts, tile);
            int local = tile - gv.tile_prefix[e];
            const int cnt = grp->counts[e], ntt = (cnt + ntok_max - 1) / ntok_max;
            const int per_mat = gv.n_row_tiles * ntt;
            const int mat = local / per_mat;
            local -= mat * per_mat;
            const int tt = local % ntt;
            const int left = cnt - tt * ntok_max;
            t.row_tile = local / ntt;
            t.valid = min(ntok_max, left);
            t.ntok = min(ntok_max, (left + 15) & ~15);
            t.x_tile = (size_t)(grp->tt_prefix[e] + tt);
            t.W = a.Wm[mat] + (size_t)e * a.expert_stride;
            t.Y = a.Ym[mat] + (size_t)(grp->offsets[e] + tt * ntok_max) * a.N;
            t.tok0 = 0;
        }
        return t;
    };

    if (warp < PWARPS) {
        // ---------------- producers: two groups of CTA_ROWS threads; group g unpacks the units
        //                  i = g, g + 2, ... (one thread per tile row), so two units are always in
        //                  the making and one group's load latency hides behind the other's work ----
        const int r = threadIdx.x % CTA_ROWS, g = threadIdx.x / CTA_ROWS;
        // prefetch distance in blocks; off when every weight tile is unpacked for several token tiles (all but the
        // first of them find the bytes in L2 anyway, and the extra instructions then only cost issue slots)
        const int pf = (grp || a.n_tok_tiles == 1) ? GEMM_PF_BLOCKS : 0;
        struct Cursor { GemmShare::Cursor c; int tile, ks; const uint8_t *rowp; const uint8_t *xb; uint32_t bb; };
        auto enter_tile = [&](Cursor &c) {   // the weight row, activation tiles and token count of c.tile
            const GemmTile t = resolve(c.tile);
            const int row = t.row_tile * CTA_ROWS + r;
            c.rowp = row < a.N ? t.W + (size_t)row * row_bytes : nullptr;
            c.xb = (const uint8_t *)a.Xb + t.x_tile * (size_t)ksteps * (size_t)b_stride;
            c.bb = (uint32_t)(t.ntok * 128);
        };
        auto advance = [&](Cursor &c, int by) {   // `by` units further in this CTA's work
            sh.advance(c.c, by);
            c.ks = c.c.ks;
            if (c.c.tile != c.tile) {
                c.tile = c.c.tile;
                enter_tile(c);
            }
        };
        Cursor ld, st;
        sh.place(ld.c, g);
        ld.tile = ld.c.tile;
        ld.ks = ld.c.ks;
        ld.rowp = nullptr;
        ld.xb = nullptr;
        ld.bb = 0;
        if (g < nunits) enter_tile(ld);
        st = ld;
        int s = g % a.stages;
        uint32_t round = g / a.stages;
        bool live = true;
        // one unit: start the loads of this thread's next unit (into the other register set; formats
        // whose raw bytes are too many registers for two sets reload the one set right after unpacking),
        // wait for the stage, unpack into it
        auto produce = [&](typename P::Raw &use, typename P::Raw &pre, int i) {
            if (P::TWO_SETS && i + 2 < nunits) {
                advance(ld, 2);
                P::load(pre, ld.rowp, nb, ld.ks, pf);
            }
            if (round > 0 && !mbar_wait_sleep(&empty_bar[s], (round - 1) & 1, 32)) {
                atomicExch(a.status, QZ_ERR_TIMEOUT);
                abort_s = 1;
                live = false;
                return;
            }
            if (*(volatile int *)&abort_s) {
                live = false;
                return;
            }
            uint8_t *As = gsm + (size_t)s * stage_bytes;
            if (r == 0) {   // the activation tile of this unit: one bulk async copy
                const uint8_t *src = st.xb + (size_t)st.ks * (size_t)b_stride;
                mbar_arrive_expect_tx(&full_bar[s], st.bb);
                tma_load_1d(As + a_bytes, src, st.bb, &full_bar[s]);
            }
            P::store(As, use, st.rowp, nb, st.ks, r, tbl);   // rows >= 128 land in the second half's tile (r * 128)
            if (!P::TWO_SETS && i + 2 < nunits) {
                advance(ld, 2);
                P::load(use, ld.rowp, nb, ld.ks, pf);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[s]);
            st = ld;
            s += 2;
            while (s >= a.stages) {
                s -= a.stages;
                round++;
            }
        };
        typename P::Raw r0, r1;
        if (g < nunits) P::load(r0, ld.rowp, nb, ld.ks, pf);
        if (P::TWO_SETS) {
            for (int i = g; i < nunits && live; i += 4) {
                produce(r0, r1, i);
                if (i + 2 < nunits && live) produce(r1, r0, i + 2);
            }
        } else {
            for (int i = g; i < nunits && live; i += 2) produce(r0, r0, i);
        }
    } else if (warp == PWARPS) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t idesc = umma_idesc_bf16(ntok_max);
            int s = 0, seg = 0;
            uint32_t round = 0;
            bool ok = true, first = true;
            GemmShare::Cursor cur;
            sh.place(cur, 0);
            for (int i = 0; i < nunits && ok; i++) {
                ok = mbar_wait(&full_bar[s], round & 1);
                if (ok && first && seg > 0) ok = mbar_wait(&acc_free_bar, (seg - 1) & 1);   // accumulator drained
                if (!ok) break;
                if (first && grp) idesc = umma_idesc_bf16(resolve(cur.tile).ntok);   // this tile's token count
                tc_fence_after();
                const uint32_t a_addr = smem_u32(gsm + (size_t)s * stage_bytes), b_addr = a_addr + a_bytes;
#pragma unroll
                for (int hf = 0; hf < HALVES; hf++) {
#pragma unroll
                    for (int k = 0; k < GEMM_KSTEP / 16; k++) {
                        // advancing K by 16 bf16 inside the swizzle atom = +32 bytes on the start address
                        tc_mma_bf16(tmem_base + (uint32_t)(hf * ntok_max), umma_desc_sw128(a_addr + hf * (GEMM_ROWS * 128) + 32 * k),
                                    umma_desc_sw128(b_addr + 32 * k), idesc, (!first || k > 0) ? 1u : 0u);
                    }
                }
                tc_commit(&empty_bar[s]);   // arrives once the MMAs above have consumed the stage
                first = false;
                if (sh.run(cur) == 1) {   // the tile's last unit in this CTA's work
                    tc_commit(&done_bar);
                    seg++;
                    first = true;
                }
                if (++s == a.stages) {
                    s = 0;
                    round++;
                }
                sh.advance(cur, 1);
            }
            if (!ok) {
                atomicExch(a.status, QZ_ERR_TIMEOUT);
                abort_s = 1;
            }
        }
    } else {
        // ---------------- epilogue: four warps per half (a warp reads TMEM lanes 32 * (warp % 4) ..),
        //                  one weight row per thread ----------------
        const int hf = (warp - PWARPS - 1) >> 2, quad = warp & 3;
        int seg = 0;
        GemmShare::Cursor cur;
        sh.place(cur, 0);
        while (cur.i < nunits) {
            const int tile = cur.tile;
            const int len = sh.run(cur);
            if (*(volatile int *)&abort_s || !mbar_wait_sleep(&done_bar, seg & 1, 500)) {
                atomicExch(a.status, QZ_ERR_TIMEOUT);
                abort_s = 1;
                break;
            }
            tc_fence_after();
            const bool whole = len == ksteps;
            const GemmTile t = resolve(tile);
            const int row = t.row_tile * CTA_ROWS + GEMM_ROWS * hf + 32 * quad + lane;
            // the tile's token count is a multiple of 16: 32 columns per round trip, then at most one group of 16
            for (int c0 = 0; c0 < t.ntok; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * quad) << 16) + (uint32_t)(hf * ntok_max + c0);
                const int nc = min(32, t.ntok - c0);
                if (nc == 32) tc_ld32(taddr, v);
                else tc_ld16(taddr, v);
                if (row < a.N && a.push.n > 0 && whole) {
                    // row-sharded: straight into every rank's window (a warp writes 32 consecutive floats per token and
                    // rank: coalesced 128-byte stores, local or over NVLink)
                    const long long base = a.push_off + (long long)(t.tok0 + c0) * a.push_ld + row;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (j < nc && c0 + j < t.valid) {
                            const float f = __uint_as_float(v[j]);
                            for (int rk = 0; rk < a.push.n; rk++) a.push.data[rk][base + (long long)j * a.push_ld] = f;
                        }
                    }
                } else if (row < a.N) {
                    float *dst = t.Y + (size_t)c0 * a.N + row;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (j < nc && c0 + j < t.valid) {
                            if (whole) dst[(size_t)j * a.N] = __uint_as_float(v[j]);
                            else atomicAdd(dst + (size_t)j * a.N, __uint_as_float(v[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free_bar);
            sh.advance(cur, len);
            seg++;
        }
    }
    if (threadIdx.x == 0 && *(volatile int *)&abort_s) {
        // gave up: let this thread's own bulk copies land before the shared memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == PWARPS) tmem_dealloc(tmem_base, tmem_cols);
    // row-sharded: all of this CTA's remote stores are issued and the CTA has met: one thread counts the CTA in, the
    // last CTA of the grid fences and publishes (a CTA that gave up does not count: the peers' bounded waits report it)
    if (a.push.n > 0 && threadIdx.x == 0 && !*(volatile int *)&abort_s) push_publish(a.push, gridDim.x, a.status, true);
}

}  // namespace qz
