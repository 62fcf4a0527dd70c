// Prefill path of the MoE block: token-sorted grouped GEMMs on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in tensor memory).
//
// Reference semantics are those of the decode kernels (MoeExperts::forward_batched,
// paramecia-model/src/qwen3_next.rs:1347-1394; the CPU arithmetic of tokio_experts.rs:157-204):
// activations quantised to Q8_K, integer block dot products, f32 scales.  A tensor-core GEMM
// over dequantised fp16/bf16 operands does NOT meet the parity bar for gate/up: an error of
// 3e-4 in silu(gate)*up flips enough int8 roundings of the re-quantised activation to put the
// block output 3e-3 away from the reference.  The gate/up GEMM therefore stays in integers:
//
//   k_gu_prefill   Q4_K gate+up.  For one 256-wide block of the reduction dimension the
//                  weight sc_j * q (0..945) is split into two byte digits, q*(sc_j & 7) and
//                  q*(sc_j >> 3), each a byte-wise product of four packed nibbles with a small
//                  scalar; two kind::i8 MMAs (u8 x s8 -> s32) per 32 weights give the exact
//                  integer block sums S = D0 + 8*D1.  The minimum term sum_j m_j * bsum_j comes
//                  from two more small MMAs over the 16 partial sums of a Q8_K block, split
//                  into digits bsum = 64*h + l.  After every block the epilogue warps read the
//                  s32 accumulators from tensor memory and add
//                  d_x * (d_w * S - dmin_w * M) to f32 accumulators in registers -- the same
//                  f32 expression the decode kernel evaluates.  silu(gate)*up is formed at the
//                  end (gate rows and up rows share one M = 128 tile) and written as f32.
//   k_down_prefill down projection over the re-quantised activation (see below).
//
// Tiles: M = 128 weight rows (64 gate + 64 up), N = 64 tokens of one expert.  Decoded weight tiles
// are staged in shared memory in the K-major core-matrix layout (8 rows x 16 bytes, no swizzle);
// token tiles arrive by TMA (cp.async.bulk.tensor, no multicast) in the 128-byte swizzled K-major
// layout: gather copies of four token rows for the Q4_K gate/up kernel, boxes of the expert-sorted
// activation array for the K-quant down kernels; the Q4_K rows' raw blocks come through tensor
// maps over the matrices as bytes.  The maps are encoded on the host with the driver's
// cuTensorMapEncodeTiled, looked up at run time.  Every wait is bounded and reports through the
// status word; tensor memory is freed on every path.
#include "pmoe_common.cuh"
#include <cstring>
#include <map>
#include <mutex>
#include <cuda.h>   // CUtensorMap and its enums; the encoder itself comes from the driver at run time

namespace pmoe {

constexpr int PF_NT = 64;        // tokens per tile (MMA N)
constexpr int PF_M = 128;        // rows per tile (MMA M): 64 gate + 64 up
constexpr int GU_REPS = 2;        // token tiles a CTA of the Q4_K gate/up kernel takes, one after the other
constexpr int GU_THREADS = 256;   // gate/up kernel: two threads per weight row (one per half of a 256-wide block)
constexpr int PF_TMEM_COLS = 256;  // D0, D1, Dh, Dl: 4 x 64 columns of s32

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ inline void tmem_alloc(uint32_t *smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_dealloc(uint32_t addr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 8-bit integer operands, s32 accumulate
__device__ inline void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ inline void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive 32-bit columns of this warp's 32 lanes
__device__ inline void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ inline void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes;
// lbo = bytes between the two 16-byte K chunks of one MMA, sbo = bytes between 8-row groups.
__device__ inline uint64_t smem_desc(const void *p, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(p) & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of this architecture
    return d;
}
// The same for the 128-byte swizzled K-major layout: a row is 128 contiguous bytes (64 halves of K) whose 16-byte
// chunks sit at chunk ^ (row & 7); 8-row groups are 1024 bytes apart; the tile starts on a 1024-byte boundary.  A K
// slice of 16 halves is 32 bytes further on in the start address.
__device__ inline uint64_t smem_desc_sw128(const void *p)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(p) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset: not used by this layout
    d |= (uint64_t)(1024 >> 4) << 32;  // stride between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version of this architecture
    d |= (uint64_t)2 << 61;            // 128-byte swizzle
    return d;
}
// Instruction descriptor: D format (1 = f32, 2 = s32) | A/B formats | N/8 | M/16; K-major A and B.
__device__ constexpr uint32_t make_idesc(uint32_t cfmt, uint32_t afmt, uint32_t bfmt, uint32_t n, uint32_t m)
{
    return (cfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// byte offset of (row, kbyte) inside a K-major core-matrix tile with `rows` rows
__device__ inline uint32_t core_off(int rows, int row, int kbyte)
{
    return (uint32_t)((kbyte >> 4) * (rows * 16) + (row >> 3) * 128 + (row & 7) * 16 + (kbyte & 15));
}

// one box of a 2-D tensor map (rows y .. y + 63, 64 halves from x on) into shared memory; the bytes count on `bar`
__device__ inline void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// four rows y0 .. y3 of a 2-D tensor map (box: one row), columns from x on, into four consecutive rows of shared memory
__device__ inline void tma_gather4(void *smem_dst, const CUtensorMap *map, int x, int y0, int y1, int y2, int y3, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
        : "memory");
}

// ---------------------------------------------------------------- gate/up, Q4_K, exact integer block sums
struct GuArgs {
    const uint8_t *gate, *up;      // routed [E_local, F, H] Q4_K
    size_t expert_bytes;
    const uint8_t *sgate, *sup;    // shared expert (may be null)
    int has_shared, routed;
    int n, top_k, H, F;
    int sh_begin, sh_count;        // tokens the shared expert serves
    Groups g;
    const int *tile_prefix;        // [n_active + 1] exclusive prefix of ceil(count / PF_NT) over active slots
    QAct xq;                       // Q8_K rows of the input [n, H]
    CUtensorMap xq_map;            // TMA descriptor of xq.qs for the Q4_K kernel: boxes of one row x 128 bytes, 128-byte swizzle
    CUtensorMap w_map[4];          // ... of gate, up, sgate, sup as [rows, row bytes / 4] words: boxes of 64 rows x one Q4_K block
                                   // (Q8_0: x eight blocks)
    CUtensorMap xd_map;            // Q8_0: ... of xq.d as [n, H / 32] floats: boxes of one row x 4 floats (a 128-wide step's scales)
    float *act;                    // [n*(k+1), F]
    DevStatus *status;
};

struct GuSmem {
    // the tile's quants of one 256-wide block: per half of the block 64 rows of 128 bytes in the 128-byte swizzled
    // K-major layout (what a gather copy of four token rows writes); on a 1024-byte boundary
    uint8_t b[2][PF_NT * 128];
    // the 128 rows' raw bytes of the current block (one Q4_K block of 144 bytes each): two TMA boxes, gate and up
    uint8_t raw[PF_M][Q4_K_BYTES];
    uint8_t a0[PF_M * 256];
    uint8_t a1[PF_M * 256];
    uint8_t am[PF_M * 32];
    uint8_t bh[PF_NT * 32];
    uint8_t bl[PF_NT * 32];
    float dx[PF_NT];
    int row_in[PF_NT];
    int row_out[PF_NT];
    uint64_t bar, bar_full, bar_raw;
    uint32_t tmem_base;
    int slot, tile_in_slot;
};
static_assert(sizeof(GuSmem) + 1024 + 128 <= 115712, "two CTAs of the gate/up GEMM share an SM");

__global__ void __launch_bounds__(GU_THREADS, 2) k_gu_prefill(const __grid_constant__ GuArgs A)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    GuSmem &S = *reinterpret_cast<GuSmem *>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which (expert slot, token tile) is this CTA's
    const int n_active = A.routed ? *A.g.n_active : 0;
    const int routed_tiles = n_active ? A.tile_prefix[n_active] : 0;
    const int shared_tiles = A.has_shared ? (A.sh_count + PF_NT - 1) / PF_NT : 0;
    const int total_tiles = routed_tiles + shared_tiles, first = blockIdx.y * GU_REPS;
    if (first >= total_tiles) return;
    if (tid == 0) {
        mbar_init(&S.bar, 1);
        mbar_init(&S.bar_full, 1);
        mbar_init(&S.bar_raw, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&S.tmem_base, PF_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = S.tmem_base;
    uint32_t phase = 0;
    bool ok = true;
    // K positions 16 .. 31 of the partial-sum digit tiles stay zero for the CTA's life (the MMA's K is 32)
    if (tid < PF_NT) {
        *reinterpret_cast<uint4 *>(S.bh + core_off(PF_NT, tid, 16)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4 *>(S.bl + core_off(PF_NT, tid, 16)) = make_uint4(0, 0, 0, 0);
    }
    // Everything a block reads from memory arrives by TMA while the block before it is under way.  The tile's quants:
    // gather copies of four token rows and one half of the block each, issued (four lanes of every warp, one
    // instruction a warp: issuing a copy is not cheap for the thread that does it) once the MMAs of the block before
    // have been waited for; padding rows of a ragged tile read row 0 (their columns are never stored).  The rows' raw
    // bytes: two boxes (64 gate rows, 64 up rows, one Q4_K block each), issued once every thread has taken its share
    // of the block before into registers.  `img` counts the CTA's blocks: the parity of both barriers.
    uint32_t img = 0;
    auto fetch_b = [&](int blk) {
        if (tid == 0) mbar_expect_tx(&S.bar_full, 2 * PF_NT * 128);
        if (lane < 4) {   // copy g = 4 warp + lane of the block's 32: rows 4 (g / 2) .. + 3, half g % 2
            const int g = 4 * warp + lane;
            const int4 rr = *reinterpret_cast<const int4 *>(&S.row_in[4 * (g >> 1)]);
            const int y0 = rr.x < 0 ? 0 : rr.x, y1 = rr.y < 0 ? 0 : rr.y, y2 = rr.z < 0 ? 0 : rr.z, y3 = rr.w < 0 ? 0 : rr.w;
            tma_gather4(&S.b[g & 1][4 * (g >> 1) * 128], &A.xq_map, blk * QK_K + 128 * (g & 1), y0, y1, y2, y3, &S.bar_full);
        }
    };
    // the CTA's tiles, one after the other: set-up (tensor memory, barrier) is paid once, and the second tile of an
    // expert finds the rows the first one read in the caches
    for (int rep = 0; rep < GU_REPS && first + rep < total_tiles && ok; rep++) {
    const int tile = first + rep;
    if (tid == 0) {
        if (tile < routed_tiles) {
            const int2 ti = A.g.tile_table[tile];  // (local expert, tile inside the expert)
            S.slot = ti.x;
            S.tile_in_slot = ti.y;
        } else {
            S.slot = -1;
            S.tile_in_slot = tile - routed_tiles;
        }
    }
    __syncthreads();
    const int slot = S.slot, t0 = S.tile_in_slot * PF_NT;
    const bool is_shared = slot < 0;
    int m;
    const int *list = nullptr;
    int wrow0;   // the tile's first row in the gate / up matrices as the tensor maps see them
    if (is_shared) {
        m = A.sh_count;
        wrow0 = blockIdx.x * 64;
    } else {
        const int e = slot;
        m = A.g.count[e];
        list = A.g.pairs + A.g.offset[e];
        wrow0 = e * A.F + blockIdx.x * 64;
    }
    const CUtensorMap *map_g = &A.w_map[is_shared ? 2 : 0], *map_u = &A.w_map[is_shared ? 3 : 1];
    auto fetch_w = [&](int blk) {   // one thread (not the one that issues the MMAs)
        if (tid == 32) {
            mbar_expect_tx(&S.bar_raw, PF_M * Q4_K_BYTES);
            tma_load_2d(&S.raw[0][0], map_g, blk * (Q4_K_BYTES / 4), wrow0, &S.bar_raw);   // (the maps count 4-byte words)
            tma_load_2d(&S.raw[64][0], map_u, blk * (Q4_K_BYTES / 4), wrow0, &S.bar_raw);
        }
    };
    const int cnt = m - t0 < PF_NT ? m - t0 : PF_NT;
    if (tid < PF_NT) {
        int rin = -1, rout = -1;
        if (tid < cnt) {
            if (is_shared) { rin = A.sh_begin + t0 + tid; rout = A.n * A.top_k + rin; }
            else { const int p = list[t0 + tid]; rin = p / A.top_k; rout = p; }
        }
        S.row_in[tid] = rin;
        S.row_out[tid] = rout;
    }
    __syncthreads();
    fetch_b(0);
    fetch_w(0);

    // this thread's weight row r: rows 0..63 are gate rows, 64..127 the up rows of the same 64 outputs.
    // Threads r and r + 128 share a row: kh = 0 decodes sub-blocks 0..3 of each block and drains
    // token columns 0..31, kh = 1 sub-blocks 4..7 and columns 32..63.
    const int r = tid & (PF_M - 1), kh = tid >> 7;
    const int f0 = blockIdx.x * 64;
    const int nblk = A.H / QK_K;

    constexpr uint32_t IDESC_UU_S = make_idesc(2, 0, 1, PF_NT, PF_M);  // u8 x s8
    constexpr uint32_t IDESC_UU_U = make_idesc(2, 0, 0, PF_NT, PF_M);  // u8 x u8
    // shared-memory descriptors of the operand tiles (the tiles do not move; a K slice is an address offset)
    const uint64_t desc_a0 = smem_desc(S.a0, PF_M * 16, 128), desc_a1 = smem_desc(S.a1, PF_M * 16, 128);
    const uint64_t desc_am = smem_desc(S.am, PF_M * 16, 128);
    const uint64_t desc_bh = smem_desc(S.bh, PF_NT * 16, 128), desc_bl = smem_desc(S.bl, PF_NT * 16, 128);
    constexpr int NC = PF_NT / 2;  // token columns this thread drains
    float acc[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) acc[i] = 0.f;

    for (int b = 0; b < nblk && ok; b++) {
        // ---- the thread's half of its row's block: header + 64 bytes of quants, from the rows the copies brought
        if (!mbar_wait_spin(&S.bar_raw, img & 1)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 32, b);
            ok = false;
        }
        uint4 blk[5];
        blk[0] = *reinterpret_cast<const uint4 *>(&S.raw[r][0]);
#pragma unroll
        for (int i = 0; i < 4; i++) blk[1 + i] = *reinterpret_cast<const uint4 *>(&S.raw[r][16 + 64 * kh + 16 * i]);
        // the tile's partial sums of 16 quants: four threads per token, four sums each (every warp takes its share of
        // this, the loads are whole sectors)
        const int tq = tid >> 2, qq = tid & 3;
        const int rin_q = S.row_in[tq];
        uint2 bsq = make_uint2(0u, 0u);
        float dx_reg = 0.f;
        if (rin_q >= 0) {
            bsq = *reinterpret_cast<const uint2 *>(A.xq.bsums + (size_t)rin_q * (A.H / 16) + b * 16 + 4 * qq);
            if (qq == 0) dx_reg = A.xq.d[(size_t)rin_q * nblk + b];
        }
        // ---- A: two digit tiles and the mins tile for this thread's row
        const uint4 hdr = blk[0];
        const float dw = half_bits_to_float((uint16_t)(hdr.x & 0xffffu));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        // 6-bit scales and mins as bytes: sc[0..3] in sca, sc[4..7] in scb, likewise mins
        const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
        const uint32_t sca = u0 & 0x3F3F3F3Fu, mna = u1 & 0x3F3F3F3Fu;
        const uint32_t scb = (u2 & 0x0F0F0F0Fu) | ((u0 >> 2) & 0x30303030u);
        const uint32_t mnb = ((u2 >> 4) & 0x0F0F0F0Fu) | ((u1 >> 2) & 0x30303030u);
        const uint32_t scw = kh == 0 ? sca : scb;   // the four scales of this thread's half
#pragma unroll
        for (int gl = 0; gl < 2; gl++) {
            const int gq = 2 * kh + gl;                // 64-weight group of the block
            const uint4 qa = blk[1 + 2 * gl], qb = blk[2 + 2 * gl];
            const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const uint32_t sc_lo = (scw >> (16 * gl)) & 0xFFu;        // sub-block 2*gq   (low nibbles)
            const uint32_t sc_hi = (scw >> (16 * gl + 8)) & 0xFFu;    // sub-block 2*gq+1 (high nibbles)
            uint32_t d0[8], d1[8], e0[8], e1[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
                d0[i] = lo * (sc_lo & 7u); d1[i] = lo * (sc_lo >> 3);
                e0[i] = hi * (sc_hi & 7u); e1[i] = hi * (sc_hi >> 3);
            }
            // sub-block j occupies K bytes 32j .. 32j+31 = chunks 2j, 2j+1
            const int j0 = 2 * gq, j1 = 2 * gq + 1;
            *reinterpret_cast<uint4 *>(S.a0 + core_off(PF_M, r, 32 * j0)) = make_uint4(d0[0], d0[1], d0[2], d0[3]);
            *reinterpret_cast<uint4 *>(S.a0 + core_off(PF_M, r, 32 * j0 + 16)) = make_uint4(d0[4], d0[5], d0[6], d0[7]);
            *reinterpret_cast<uint4 *>(S.a1 + core_off(PF_M, r, 32 * j0)) = make_uint4(d1[0], d1[1], d1[2], d1[3]);
            *reinterpret_cast<uint4 *>(S.a1 + core_off(PF_M, r, 32 * j0 + 16)) = make_uint4(d1[4], d1[5], d1[6], d1[7]);
            *reinterpret_cast<uint4 *>(S.a0 + core_off(PF_M, r, 32 * j1)) = make_uint4(e0[0], e0[1], e0[2], e0[3]);
            *reinterpret_cast<uint4 *>(S.a0 + core_off(PF_M, r, 32 * j1 + 16)) = make_uint4(e0[4], e0[5], e0[6], e0[7]);
            *reinterpret_cast<uint4 *>(S.a1 + core_off(PF_M, r, 32 * j1)) = make_uint4(e1[0], e1[1], e1[2], e1[3]);
            *reinterpret_cast<uint4 *>(S.a1 + core_off(PF_M, r, 32 * j1 + 16)) = make_uint4(e1[4], e1[5], e1[6], e1[7]);
        }
        if (kh == 0) {   // mins, each repeated for the two 16-wide halves of its sub-block: m0 m0 m1 m1 ... m7 m7, then zeros
            const uint32_t w0 = __byte_perm(mna, 0, 0x1100), w1 = __byte_perm(mna, 0, 0x3322);
            const uint32_t w2 = __byte_perm(mnb, 0, 0x1100), w3 = __byte_perm(mnb, 0, 0x3322);
            *reinterpret_cast<uint4 *>(S.am + core_off(PF_M, r, 0)) = make_uint4(w0, w1, w2, w3);
            *reinterpret_cast<uint4 *>(S.am + core_off(PF_M, r, 16)) = make_uint4(0, 0, 0, 0);
        }
        {   // partial sums as two digits: bsum = 64*h + l, l in [0,63]; K positions 4 qq .. 4 qq + 3 of token tq
            uint32_t hw = 0, lw = 0;
            const uint32_t bw[2] = {bsq.x, bsq.y};   // 4 x int16
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int v = (int)(int16_t)(bw[i >> 1] >> (16 * (i & 1)));
                hw |= (uint32_t)((v >> 6) & 0xFF) << (8 * i);
                lw |= (uint32_t)(v & 63) << (8 * i);
            }
            *reinterpret_cast<uint32_t *>(S.bh + core_off(PF_NT, tq, 4 * qq)) = hw;
            *reinterpret_cast<uint32_t *>(S.bl + core_off(PF_NT, tq, 4 * qq)) = lw;
            if (qq == 0) S.dx[tq] = dx_reg;
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (b + 1 < nblk) fetch_w(b + 1);   // every thread has its share of this block's rows in registers
        // ---- MMAs of this block, issued by one thread
        if (tid == 0) {
            fence_proxy_async();   // everyone's stores are ordered before the barrier; the issuing thread crosses over to the async proxy
            tc_fence_after();
            if (!mbar_wait_spin(&S.bar_full, img & 1)) set_status(A.status, PMOE_ERR_TIMEOUT, 31, b);   // (the MMAs then run on what is there; the status word says so)
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {  // 32 bytes of K per instruction: A two 16-byte chunks further on per step, B 32 bytes inside its half's swizzled rows
                const uint64_t ka = (uint64_t)(ks * ((2 * PF_M * 16) >> 4));
                const uint64_t db = smem_desc_sw128(S.b[ks >> 2]) + (uint64_t)((ks & 3) * (32 >> 4));
                mma_i8(tmem + 0, desc_a0 + ka, db, IDESC_UU_S, ks > 0);
                mma_i8(tmem + 64, desc_a1 + ka, db, IDESC_UU_S, ks > 0);
            }
            mma_i8(tmem + 128, desc_am, desc_bh, IDESC_UU_S, 0);
            mma_i8(tmem + 192, desc_am, desc_bl, IDESC_UU_U, 0);
            tc_commit(&S.bar);
        }
        if (!mbar_wait_spin(&S.bar, phase)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 30, b);
            ok = false;
        }
        phase ^= 1;
        tc_fence_after();
        if (ok && b + 1 < nblk) fetch_b(b + 1);   // the MMAs that read the tile are done
        // ---- fold the block into the f32 accumulators: row r = TMEM lane r (a warp reaches the 32
        // lanes of its quarter, warp % 4), this thread's half of the token columns
        if (ok) {
            const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kh * NC;
#pragma unroll
            for (int cc = 0; cc < NC / 16; cc++) {
                uint32_t v0[16], v1[16], vh[16], vl[16];
                tmem_ld16(lane_addr + 0 + cc * 16, v0);
                tmem_ld16(lane_addr + 64 + cc * 16, v1);
                tmem_ld16(lane_addr + 128 + cc * 16, vh);
                tmem_ld16(lane_addr + 192 + cc * 16, vl);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int s = (int)v0[j] + 8 * (int)v1[j];
                    const int mm = 64 * (int)vh[j] + (int)vl[j];
                    acc[cc * 16 + j] += S.dx[kh * NC + cc * 16 + j] * (dw * (float)s - dmin * (float)mm);
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);  // operands and accumulators are free for the next block; a thread that gave up takes the CTA with it
        tc_fence_after();
        img++;
    }

    // ---- silu(gate) * up: all rows hand their sums over through shared memory ([128][PF_NT + 1]
    // floats over the digit tiles, which no MMA reads any more), then every thread takes a share
    // of the 64 x PF_NT outputs: output o = (token j, column f), consecutive threads = consecutive f.
    float *xch = reinterpret_cast<float *>(S.a0);
#pragma unroll
    for (int j = 0; j < NC; j++) xch[r * (PF_NT + 1) + kh * NC + j] = acc[j];
    __syncthreads();
    if (ok) {
        // thread: column f = tid & 63 of tokens (tid >> 6) + 4 i; four tokens at a time, so that their exponentials
        // and divisions overlap
        const int f = tid & 63;
        const float *xg = xch + f * (PF_NT + 1), *xu = xch + (64 + f) * (PF_NT + 1);
#pragma unroll 1
        for (int j0 = tid >> 6; j0 < PF_NT; j0 += 16) {
            float v[4];
            int rout[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = j0 + 4 * i;
                rout[i] = S.row_out[j];
                const float g = xg[j], u = xu[j];
                v[i] = g / (1.f + expf(-g)) * u;
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (rout[i] >= 0) A.act[(size_t)rout[i] * A.F + f0 + f] = v[i];
        }
    }
    tc_fence_before();
    __syncthreads();   // tiles, tables and accumulators are free for the CTA's next tile
    tc_fence_after();
    }
    // a CTA that gave up may have a block's copies under way: they land (bounded wait) before its shared memory goes
    if (!ok && tid == 0) {
        mbar_wait(&S.bar_full, img & 1, 1u << 8);
        mbar_wait(&S.bar_raw, img & 1, 1u << 8);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, PF_TMEM_COLS);
}

// ---------------------------------------------------------------- gate/up, Q8_0, exact integer block sums
// Q8_0 weights against Q8_0 activations (what the reference CPU path does for this type): one block of 32 is the
// K of one kind::i8 MMA (s8 x s8 -> s32), and every block has its own accumulator -- four blocks (K = 128) per
// step fill 4 x 64 columns of tensor memory -- because the scales d_w (per row and block) and d_x (per token and
// block) meet the integer sum only afterwards: acc += (d_w * d_x) * S, exactly the f32 expression of the decode
// kernels, block after block in K order.  The weights need no decoding: a thread copies its row's quants into the
// K-major core-matrix layout (the 34-byte blocks put every second block's quants 2 bytes off a word: funnel shifts).
struct Gu80Ops {
    uint8_t a[PF_M * 128];          // the rows' quants of one step, core-matrix layout
    uint8_t b[PF_NT * 128];         // the tokens' quants of one step: 64 rows of 128 bytes, 128-byte swizzle (gather copies)
    float dw[4][PF_M];
};
struct Gu80Smem {
    union {
        Gu80Ops o;                           // operands and scales of one step (on a 1024-byte boundary)
        float xch[PF_M * (PF_NT + 1)];       // the accumulators' way to silu(gate) * up at the end
    };
    // the rows' raw bytes, two steps (eight blocks, 272 bytes a row) at a time, double-buffered: two TMA boxes (64 gate
    // rows, 64 up rows) per chunk
    uint8_t raw[2][PF_M][8 * Q8_0_BYTES];
    // the tokens' four scales of a step, two steps: a gather copy brings four tokens' scales (64 bytes) and wants a
    // 128-byte aligned destination, so every group of four tokens has a 128-byte slot of which it fills half
    float dx[2][PF_NT / 4][32];
    int row_in[PF_NT];
    int row_out[PF_NT];
    uint64_t bar, bar_raw[2], bar_full;
    uint32_t tmem_base;
    int slot, tile_in_slot;
};
static_assert(sizeof(Gu80Smem) + 1024 + 128 <= 115712, "two CTAs of the Q8_0 gate/up GEMM share an SM");
static_assert((8 * Q8_0_BYTES) % 16 == 0, "TMA boxes need rows of a multiple of 16 bytes");

__global__ void __launch_bounds__(GU_THREADS, 2) k_gu_prefill_q80(const __grid_constant__ GuArgs A)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Gu80Smem &S = *reinterpret_cast<Gu80Smem *>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int n_active = A.routed ? *A.g.n_active : 0;
    const int routed_tiles = n_active ? A.tile_prefix[n_active] : 0;
    const int shared_tiles = A.has_shared ? (A.sh_count + PF_NT - 1) / PF_NT : 0;
    const int tile = blockIdx.y;
    if (tile >= routed_tiles + shared_tiles) return;
    if (tid == 0) {
        if (tile < routed_tiles) {
            const int2 ti = A.g.tile_table[tile];
            S.slot = ti.x;
            S.tile_in_slot = ti.y;
        } else {
            S.slot = -1;
            S.tile_in_slot = tile - routed_tiles;
        }
        mbar_init(&S.bar, 1);
        mbar_init(&S.bar_raw[0], 1);
        mbar_init(&S.bar_raw[1], 1);
        mbar_init(&S.bar_full, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&S.tmem_base, PF_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = S.tmem_base;
    const int slot = S.slot, t0 = S.tile_in_slot * PF_NT;
    const bool is_shared = slot < 0;
    int m;
    const int *list = nullptr;
    int wrow0;   // the tile's first row in the gate / up matrices as the tensor maps see them
    if (is_shared) {
        m = A.sh_count;
        wrow0 = blockIdx.x * 64;
    } else {
        m = A.g.count[slot];
        list = A.g.pairs + A.g.offset[slot];
        wrow0 = slot * A.F + blockIdx.x * 64;
    }
    const CUtensorMap *map_g = &A.w_map[is_shared ? 2 : 0], *map_u = &A.w_map[is_shared ? 3 : 1];
    const int cnt = m - t0 < PF_NT ? m - t0 : PF_NT;
    if (tid < PF_NT) {
        int rin = -1, rout = -1;
        if (tid < cnt) {
            if (is_shared) { rin = A.sh_begin + t0 + tid; rout = A.n * A.top_k + rin; }
            else { const int p = list[t0 + tid]; rin = p / A.top_k; rout = p; }
        }
        S.row_in[tid] = rin;
        S.row_out[tid] = rout;
    }
    __syncthreads();

    // thread (r, kh): weight row r (0..63 gate, 64..127 up), blocks 2 kh and 2 kh + 1 of every 128-wide step;
    // afterwards it drains token columns 32 kh .. 32 kh + 31 of row r
    const int r = tid & (PF_M - 1), kh = tid >> 7;
    const int f0 = blockIdx.x * 64;
    const int steps = A.H / 128;

    constexpr uint32_t IDESC_SS = make_idesc(2, 1, 1, PF_NT, PF_M);  // s8 x s8 -> s32
    const uint64_t desc_a = smem_desc(S.o.a, PF_M * 16, 128), desc_b = smem_desc_sw128(S.o.b);
    constexpr int NC = PF_NT / 2;
    float acc[NC];
#pragma unroll
    for (int i = 0; i < NC; i++) acc[i] = 0.f;
    uint32_t phase = 0;
    bool ok = true;

    // the thread's two blocks of the current step: 68 bytes from a 4-byte boundary
    //   [0,2) d of block 0 | [2,34) its quants | [34,36) d of block 1 | [36,68) its quants
    // chunk c = steps 2c, 2c + 1 of all 128 rows -> raw[c & 1]; its barrier completes for the (c >> 1)-th time
    constexpr int CHUNK = 8 * Q8_0_BYTES;
    const int chunks = steps / 2;
    auto fetch_chunk = [&](int c) {
        if (tid == 32) {   // (not the thread that issues the MMAs)
            mbar_expect_tx(&S.bar_raw[c & 1], PF_M * CHUNK);
            tma_load_2d(&S.raw[c & 1][0][0], map_g, c * (CHUNK / 4), wrow0, &S.bar_raw[c & 1]);   // (the maps count 4-byte words)
            tma_load_2d(&S.raw[c & 1][64][0], map_u, c * (CHUNK / 4), wrow0, &S.bar_raw[c & 1]);
        }
    };
    // The tokens' side of step s: their quants (64 rows of 128 bytes) and their four scales, by gather copies of four
    // token rows each, one instruction per warp (lanes 0..3: copy g = 4 warp + lane; the first sixteen bring quants,
    // the others scales); padding rows of a ragged tile read row 0, their columns are never stored.  Issued when the
    // MMAs of step s - 1 are done; the scales have two buffers, since the drain of step s - 1 still reads its own.
    auto fetch_x = [&](int s_) {
        if (tid == 0) mbar_expect_tx(&S.bar_full, PF_NT * 128 + PF_NT * 16);
        if (lane < 4) {
            const int g = 4 * warp + lane, grp = g & 15;
            const int4 rr = *reinterpret_cast<const int4 *>(&S.row_in[4 * grp]);
            const int y0 = rr.x < 0 ? 0 : rr.x, y1 = rr.y < 0 ? 0 : rr.y, y2 = rr.z < 0 ? 0 : rr.z, y3 = rr.w < 0 ? 0 : rr.w;
            if (g < 16) tma_gather4(&S.o.b[4 * grp * 128], &A.xq_map, 128 * s_, y0, y1, y2, y3, &S.bar_full);
            else tma_gather4(&S.dx[s_ & 1][grp][0], &A.xd_map, 4 * s_, y0, y1, y2, y3, &S.bar_full);
        }
    };
    fetch_x(0);
    fetch_chunk(0);
    if (chunks > 1) fetch_chunk(1);
    int chunks_seen = 0, chunks_issued = chunks > 1 ? 2 : 1;
    uint32_t raw[17];
    for (int s = 0; s < steps && ok; s++) {
        if ((s & 1) == 0) {
            const int c = s >> 1;
            // the buffer chunk c - 1 sat in is free: its last readers passed the barrier that ended step s - 1
            if (c >= 1 && c + 1 < chunks) { fetch_chunk(c + 1); chunks_issued = c + 2; }
            if (!mbar_wait(&S.bar_raw[c & 1], (uint32_t)((c >> 1) & 1))) {   // (the vote below takes the CTA out as one)
                set_status(A.status, PMOE_ERR_TIMEOUT, 36, c);
                ok = false;
            } else {
                chunks_seen = c + 1;
            }
        }
        {   // this thread's two blocks: 68 bytes, 4-byte aligned (a step starts on an 8-byte boundary)
            const uint8_t *p = S.raw[(s >> 1) & 1][r] + 136 * (s & 1) + 68 * kh;
            if (kh == 0) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint2 v = reinterpret_cast<const uint2 *>(p)[i];
                    raw[2 * i] = v.x; raw[2 * i + 1] = v.y;
                }
                raw[16] = *reinterpret_cast<const uint32_t *>(p + 64);
            } else {
                raw[0] = *reinterpret_cast<const uint32_t *>(p);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint2 v = reinterpret_cast<const uint2 *>(p + 4)[i];
                    raw[1 + 2 * i] = v.x; raw[2 + 2 * i] = v.y;
                }
            }
        }
        // ---- A: the row's two blocks of quants
        {
            uint32_t q0[8];
#pragma unroll
            for (int i = 0; i < 8; i++) q0[i] = __funnelshift_r(raw[i], raw[i + 1], 16);
            const int kb0 = 64 * kh;   // K byte of block 2 kh inside the step
            *reinterpret_cast<uint4 *>(S.o.a + core_off(PF_M, r, kb0)) = make_uint4(q0[0], q0[1], q0[2], q0[3]);
            *reinterpret_cast<uint4 *>(S.o.a + core_off(PF_M, r, kb0 + 16)) = make_uint4(q0[4], q0[5], q0[6], q0[7]);
            *reinterpret_cast<uint4 *>(S.o.a + core_off(PF_M, r, kb0 + 32)) = make_uint4(raw[9], raw[10], raw[11], raw[12]);
            *reinterpret_cast<uint4 *>(S.o.a + core_off(PF_M, r, kb0 + 48)) = make_uint4(raw[13], raw[14], raw[15], raw[16]);
            S.o.dw[2 * kh][r] = half_bits_to_float((uint16_t)(raw[0] & 0xffffu));
            S.o.dw[2 * kh + 1][r] = half_bits_to_float((uint16_t)(raw[8] >> 16));
        }
        // ---- the tokens' side must have landed (every thread looks: the drain reads the scales)
        if (!mbar_wait_spin(&S.bar_full, (uint32_t)(s & 1))) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 37, s);
            ok = false;
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (tid == 0) {
            fence_proxy_async();   // everyone's stores are ordered before the barrier; the issuing thread crosses over to the async proxy
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < 4; j++)   // one block = 32 bytes of K = one instruction, its own 64 columns
                mma_i8(tmem + 64 * j, desc_a + (uint64_t)(j * ((2 * PF_M * 16) >> 4)), desc_b + (uint64_t)(j * (32 >> 4)), IDESC_SS, 0);
            tc_commit(&S.bar);
        }
        if (!mbar_wait_spin(&S.bar, phase)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 35, s);
            ok = false;
        }
        phase ^= 1;
        tc_fence_after();
        if (ok && s + 1 < steps) fetch_x(s + 1);   // the MMAs that read the tile are done
        if (ok) {
            const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kh * NC;
            const float dw0 = S.o.dw[0][r], dw1 = S.o.dw[1][r], dw2 = S.o.dw[2][r], dw3 = S.o.dw[3][r];
#pragma unroll
            for (int cc = 0; cc < NC / 16; cc++) {
                uint32_t v0[16], v1[16], v2[16], v3[16];
                tmem_ld16(lane_addr + 0 + cc * 16, v0);
                tmem_ld16(lane_addr + 64 + cc * 16, v1);
                tmem_ld16(lane_addr + 128 + cc * 16, v2);
                tmem_ld16(lane_addr + 192 + cc * 16, v3);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 16; t++) {   // a token's sum takes the step's four blocks in K order
                    const int tk = kh * NC + cc * 16 + t;
                    const float4 dx = *reinterpret_cast<const float4 *>(&S.dx[s & 1][tk >> 2][4 * (tk & 3)]);
                    float a = acc[cc * 16 + t];
                    a += (dw0 * dx.x) * (float)(int)v0[t];
                    a += (dw1 * dx.y) * (float)(int)v1[t];
                    a += (dw2 * dx.z) * (float)(int)v2[t];
                    a += (dw3 * dx.w) * (float)(int)v3[t];
                    acc[cc * 16 + t] = a;
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);  // operands, scales and accumulators are free for the next step
        tc_fence_after();
    }

    // ---- silu(gate) * up through shared memory ([128][PF_NT + 1] floats, over the operand tiles and the scale
    // arrays, which nothing reads any more)
    float *xch = S.xch;
#pragma unroll
    for (int j = 0; j < NC; j++) xch[r * (PF_NT + 1) + kh * NC + j] = acc[j];
    __syncthreads();
    if (ok) {
        // thread: column f = tid & 63 of tokens (tid >> 6) + 4 i; four tokens at a time, so that their exponentials
        // and divisions overlap
        const int f = tid & 63;
        const float *xg = xch + f * (PF_NT + 1), *xu = xch + (64 + f) * (PF_NT + 1);
#pragma unroll 1
        for (int j0 = tid >> 6; j0 < PF_NT; j0 += 16) {
            float v[4];
            int rout[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = j0 + 4 * i;
                rout[i] = S.row_out[j];
                const float g = xg[j], u = xu[j];
                v[i] = g / (1.f + expf(-g)) * u;
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (rout[i] >= 0) A.act[(size_t)rout[i] * A.F + f0 + f] = v[i];
        }
    }
    if (!ok && tid == 0) {   // gave up somewhere: copies may still be on their way into this CTA's shared memory
        for (int c = chunks_seen; c < chunks_issued; c++) mbar_wait(&S.bar_raw[c & 1], (uint32_t)((c >> 1) & 1), 1u << 8);
        mbar_wait(&S.bar_full, 0, 1u << 8);
        mbar_wait(&S.bar_full, 1, 1u << 8);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, PF_TMEM_COLS);
}

// ---------------------------------------------------------------- down projection, fp16 operands
// The down GEMM has no re-quantisation after it, so its own rounding lands in the output
// directly: dequantised fp16 weights times the fake-quantised activation d*q in fp16 with f32
// accumulation in tensor memory stays near 3e-4 of the integer result, inside the parity bar.
// Tile: M = 128 output rows, N = 64 tokens, K walked in steps of 128.  The raw GGUF rows of the
// tile arrive with one bulk (TMA) copy; each thread dequantises its own row straight into the
// K-major core-matrix layout.
struct DownArgs {
    const uint8_t *down;           // routed [E_local, H, F]
    size_t expert_bytes;
    const uint8_t *sdown;          // shared
    int has_shared, routed;
    int n, top_k, H, F;
    int sh_begin, sh_count;
    Groups g;
    const int *tile_prefix;
    const __half *act_h;           // [n*(k+1), F] fake-quantised activation, routed rows in expert-sorted order
    CUtensorMap act_map;           // its TMA descriptor: boxes of 64 rows x 64 halves, 128-byte swizzle
    const float *act_h_scale;      // [n*(k+1)] power of two each row of act_h was divided by
    const float *scale_r;          // routing weights [n*k]
    const float *scale_s;          // shared gate [n]
    float *partial;                // [n*(k+1), H]
    DevStatus *status;
};

constexpr int DN_KSTEP = 64;

// 4 unsigned bytes -> 4 halves holding (byte - bias) * s
__device__ inline void bytes_to_half4(uint32_t v, __half2 bias, __half2 s, uint32_t &o0, uint32_t &o1)
{
    // 0x6400 | b is the fp16 number 1024 + b, exactly
    const uint32_t p0 = __byte_perm(v, 0x64646464u, 0x4140), p1 = __byte_perm(v, 0x64646464u, 0x4342);
    const __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&p0), bias), s);
    const __half2 h1 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&p1), bias), s);
    o0 = *reinterpret_cast<const uint32_t *>(&h0);
    o1 = *reinterpret_cast<const uint32_t *>(&h1);
}

// step(row, s, a_tile, r, part): weights 64 s .. 64 s + 63 of raw row `row` as fp16 into row r of the A tile
// (core-matrix layout, K index inside the step); two threads share a row, `part` says which half of the work
template <int DT> struct DownDequant;

// Q6_K: step s = quads 2 (s & 1), 2 (s & 1) + 1 of half (s >> 1) & 1 of block s >> 2.  In a half, quad q's weight l
// (0..31) has its low nibble in ql[l + 32 (q & 1)] (the high nibble for q >= 2) and bits 2q, 2q+1 of qh[l].
template <> struct DownDequant<PMOE_Q6_K> {
    static constexpr int ROW_BYTES = 2 * Q6_K_BYTES;  // F = 512
    __device__ static inline void step(const uint8_t *row, int s, uint8_t *a_tile, int r, int part)
    {
        const uint8_t *blk = row + (s >> 2) * Q6_K_BYTES;
        const int half = (s >> 1) & 1, qp = s & 1;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 208));
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * half + 4 * qp);
        const __half2 bias = __floats2half2_rn(1056.f, 1056.f);  // 1024 + 32
#pragma unroll
        for (int l8i = 0; l8i < 2; l8i++) {  // l = 8*l8 .. 8*l8+7
            const int l8 = 2 * part + l8i;
            const uint8_t *ql = blk + 64 * half + 8 * l8, *qh = blk + 128 + 32 * half + 8 * l8;
            uint32_t la0 = lds_u32_a2(ql), la1 = lds_u32_a2(ql + 4), lb0 = lds_u32_a2(ql + 32), lb1 = lds_u32_a2(ql + 36);
            uint32_t h0 = lds_u32_a2(qh), h1 = lds_u32_a2(qh + 4);
            if (qp) { la0 >>= 4; la1 >>= 4; lb0 >>= 4; lb1 >>= 4; h0 >>= 2; h1 >>= 2; }
            else { h0 <<= 2; h1 <<= 2; }
            // now: quad 2qp+1 has its two high bits at bits 4,5 of h; quad 2qp two places lower
            const int is = l8 >> 1;  // l / 16
#pragma unroll
            for (int qq = 0; qq < 2; qq++) {
                const float sf = d * (float)sc[is + 2 * qq];
                const __half2 sh = __floats2half2_rn(sf, sf);
                const uint32_t va = ((qq ? lb0 : la0) & 0x0F0F0F0Fu) | ((qq ? h0 : h0 << 2) & 0x30303030u);
                const uint32_t vb = ((qq ? lb1 : la1) & 0x0F0F0F0Fu) | ((qq ? h1 : h1 << 2) & 0x30303030u);
                uint4 o;
                bytes_to_half4(va, bias, sh, o.x, o.y);
                bytes_to_half4(vb, bias, sh, o.z, o.w);
                *reinterpret_cast<uint4 *>(a_tile + core_off(PF_M, r, 2 * (32 * qq + 8 * l8))) = o;
            }
        }
    }
};

// Q4_K: step s = sub-blocks 2 (s & 3), 2 (s & 3) + 1 of block s >> 2: the low and the high nibbles of 32 bytes
template <> struct DownDequant<PMOE_Q4_K> {
    static constexpr int ROW_BYTES = 2 * Q4_K_BYTES;
    __device__ static inline void step(const uint8_t *row, int s, uint8_t *a_tile, int r, int part)
    {
        const uint8_t *blk = row + (s >> 2) * Q4_K_BYTES;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        const float d = half_bits_to_float((uint16_t)(hdr.x & 0xffffu));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        const uint32_t u0 = hdr.y, u1 = hdr.z, u2 = hdr.w;
        const int upper = (s >> 1) & 1, gq = s & 1;   // sub-blocks 4..7 keep their scales in the packed form
        const uint32_t scw = upper ? (u2 & 0x0F0F0F0Fu) | ((u0 >> 2) & 0x30303030u) : u0 & 0x3F3F3F3Fu;
        const uint32_t mnw = upper ? ((u2 >> 4) & 0x0F0F0F0Fu) | ((u1 >> 2) & 0x30303030u) : u1 & 0x3F3F3F3Fu;
        // this thread: bytes 16 part .. 16 part + 15 of the 32 = weights 16 part .. + 15 of both sub-blocks
        const uint4 q = *reinterpret_cast<const uint4 *>(blk + 16 + 64 * upper + 32 * gq + 16 * part);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            const int j = 2 * gq + hi;  // sub-block inside its group of four
            const float sf = d * (float)((scw >> (8 * j)) & 0xFFu);
            const float mf = dmin * (float)((mnw >> (8 * j)) & 0xFFu);
#pragma unroll
            for (int ci = 0; ci < 2; ci++) {  // 8 weights per 16-byte chunk
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint32_t v = hi ? (w[2 * ci + i] >> 4) & 0x0F0F0F0Fu : w[2 * ci + i] & 0x0F0F0F0Fu;
                    const __half2 a = __floats2half2_rn(fmaf(sf, (float)(v & 0xFF), -mf), fmaf(sf, (float)((v >> 8) & 0xFF), -mf));
                    const __half2 bq = __floats2half2_rn(fmaf(sf, (float)((v >> 16) & 0xFF), -mf), fmaf(sf, (float)(v >> 24), -mf));
                    o[2 * i] = *reinterpret_cast<const uint32_t *>(&a);
                    o[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&bq);
                }
                const int kel = 32 * hi + 16 * part + 8 * ci;
                *reinterpret_cast<uint4 *>(a_tile + core_off(PF_M, r, 2 * kel)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
};

// Q8_0: step s = blocks 2 s, 2 s + 1 of the row (F = 512: 16 blocks of 34 bytes), one per thread of the pair
template <> struct DownDequant<PMOE_Q8_0> {
    static constexpr int ROW_BYTES = 16 * Q8_0_BYTES;
    __device__ static inline void step(const uint8_t *row, int s, uint8_t *a_tile, int r, int part)
    {
        const uint8_t *blk = row + (2 * s + part) * Q8_0_BYTES;   // 2-byte aligned
        const __half d = __ushort_as_half(*reinterpret_cast<const uint16_t *>(blk));
        const __half2 d2 = __halves2half2(d, d);
        const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
        for (int c = 0; c < 4; c++) {   // 8 weights per 16-byte chunk
            uint4 o;
            // 0x6400 | (b ^ 0x80) is the fp16 number 1024 + 128 + q for the signed byte q
            bytes_to_half4(lds_u32_a2(blk + 2 + 8 * c) ^ 0x80808080u, bias, d2, o.x, o.y);
            bytes_to_half4(lds_u32_a2(blk + 6 + 8 * c) ^ 0x80808080u, bias, d2, o.z, o.w);
            *reinterpret_cast<uint4 *>(a_tile + core_off(PF_M, r, 2 * (32 * part + 8 * c))) = o;
        }
    }
};

// A CTA takes one block of 128 output rows and up to DN_TILES consecutive entries of the tile table (token tiles of
// 64).  Entries of the same expert form a run: the run's raw GGUF rows arrive with one bulk copy, every K step
// dequantises them ONCE (two threads per row) and feeds all the run's token tiles, each with its own 64 columns of
// f32 in tensor memory -- a hot expert's weights are not decoded once per token tile.  The B tiles go through a ring
// of buffers, each loaded into registers one piece ahead and stored in the core-matrix layout.  Two CTAs share an SM
// (half of tensor memory and of shared memory each), so that one's copies, dequantisation and drain overlap the
// other's MMAs.
constexpr int DN_THREADS = 256;
constexpr int DN_TILES = 4;      // 4 x 64 columns = half of tensor memory
constexpr int DN_COLS = 64 * DN_TILES;

// A B piece holds all four token tiles of a run (256 tokens: one MMA of N = 64 .. 256 per K slice) in a single buffer:
// a step is then one wait, one dequantisation, one store of the piece, one barrier.  Q8_0 rows are the widest and
// leave room for 128-token pieces only.
// The K-quant kernels fetch their pieces (128 tokens, two buffers) with TMA tensor copies straight into the swizzled
// layout, a piece ahead, and a step has one barrier (for the dequantised A tile); the Q8_0 kernel, whose rows leave
// room for one buffer only, loads its piece into registers a piece ahead and stores it.
template <int DT> struct DownCfg {
    static constexpr bool TMA_B = DT != PMOE_Q8_0;
    static constexpr int PT = 2 * PF_NT;                                 // tokens of a B piece
    static constexpr int NB = TMA_B ? 2 : 1;                             // B buffers
    static constexpr int THREADS = DN_THREADS + (TMA_B ? 32 : 0);        // the copy warp comes after the eight working warps
};

struct DownSmemHdr {
    float scale[DN_TILES][PF_NT];
    int row_in[DN_TILES][PF_NT];    // the pair (or shared-expert row) a token's output goes to, -1: none
    int row_act[DN_TILES][PF_NT];   // the row of act_h its activation sits in
    int2 entry[DN_TILES];          // (slot or -1 for the shared expert, tile inside the expert)
    uint64_t bar_raw, bar_b[4], bar_full[4];
    uint32_t tmem_base;
    int n_entries;
};

template <int DT>
__global__ void __launch_bounds__(DownCfg<DT>::THREADS, 2) k_down_prefill(const __grid_constant__ DownArgs A)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    using DQ = DownDequant<DT>;
    constexpr int NB = DownCfg<DT>::NB;
    constexpr int RAW_BYTES = PF_M * DQ::ROW_BYTES;
    constexpr int PT = DownCfg<DT>::PT, TPP = PT / PF_NT;        // tokens and token tiles of a B piece
    constexpr int LPT = PT / 32;                                 // B side: tokens of a thread (eight threads share a token)
    constexpr int B_BYTES = PT * DN_KSTEP * 2;
    // B tiles first, on a 1024-byte boundary (their swizzled layout wants it)
    uint8_t *b_tile = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // NB x [PT tokens][64 K] fp16, 128-byte swizzle
    uint8_t *a_tile = b_tile + NB * B_BYTES;                     // [128 rows][64 K] fp16, core-matrix layout
    uint8_t *raw = a_tile + PF_M * DN_KSTEP * 2;                 // the run's GGUF rows
    DownSmemHdr &S = *reinterpret_cast<DownSmemHdr *>(raw + ((RAW_BYTES + 127) / 128) * 128);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int n_active = A.routed ? *A.g.n_active : 0;
    const int routed_tiles = n_active ? A.tile_prefix[n_active] : 0;
    const int shared_tiles = A.has_shared ? (A.sh_count + PF_NT - 1) / PF_NT : 0;
    const int first = blockIdx.y * DN_TILES;
    if (first >= routed_tiles + shared_tiles) return;
    if (tid < DN_TILES) {
        const int tile = first + tid;
        int2 e = make_int2(-2, 0);
        if (tile < routed_tiles) e = A.g.tile_table[tile];
        else if (tile < routed_tiles + shared_tiles) e = make_int2(-1, tile - routed_tiles);
        S.entry[tid] = e;
    }
    if (tid == 0) {
        const int left = routed_tiles + shared_tiles - first;
        S.n_entries = left < DN_TILES ? left : DN_TILES;
        mbar_init(&S.bar_raw, 1);
        for (int i = 0; i < NB; i++) mbar_init(&S.bar_b[i], 1);
        for (int i = 0; i < 4; i++) mbar_init(&S.bar_full[i], 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(&S.tmem_base, DN_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = S.tmem_base;
    const int n_entries = S.n_entries;
    const int h0 = blockIdx.x * PF_M;
    const int steps = A.F / DN_KSTEP;
    const int r = tid & (PF_M - 1), part = tid >> 7;               // dequantisation: row and half of the step
    const int tk0 = tid >> 3, chunk = tid & 7;                     // B side: chunk `chunk` of tokens tk0 + 32 j: a warp reads four whole rows
    const uint64_t desc_a0 = smem_desc(a_tile, PF_M * 16, 128), desc_b0 = smem_desc_sw128(b_tile);

    // MMA commits are counted over the CTA's life: commit c lands on barrier c % NB as its (c / NB)-th completion
    int committed = 0, seen = 0;
    uint32_t ph_raw = 0;
    bool ok = true;
    // waits until the first `upto` commits (the MMAs they cover and everything issued before) have finished
    auto wait_mma = [&](int upto) {
        for (; seen < upto; seen++)
            if (ok && !mbar_wait_spin(&S.bar_b[seen % NB], (uint32_t)((seen / NB) & 1))) {
                set_status(A.status, PMOE_ERR_TIMEOUT, 32, seen);
                ok = false;
            }
    };

    for (int e0 = 0; e0 < n_entries && ok;) {
        const int slot = S.entry[e0].x;
        int e1 = e0 + 1;
        while (e1 < n_entries && S.entry[e1].x == slot) e1++;
        const int T = e1 - e0;                                     // token tiles of this run
        const bool is_shared = slot < 0;
        int m;
        const int *list = nullptr;
        const uint8_t *wd;
        if (is_shared) {
            m = A.sh_count;
            wd = A.sdown;
        } else {
            m = A.g.count[slot];
            list = A.g.pairs + A.g.offset[slot];
            wd = A.down + (size_t)slot * A.expert_bytes;
        }
        if (tid == 0) {   // the run's raw rows: one contiguous range
            mbar_expect_tx(&S.bar_raw, RAW_BYTES);
            const uint8_t *src = wd + (size_t)h0 * DQ::ROW_BYTES;
            for (int off = 0; off < RAW_BYTES; off += 16384)
                bulk_g2s(raw + off, src + off, RAW_BYTES - off < 16384 ? RAW_BYTES - off : 16384, &S.bar_raw);
        }
        for (int i = tid; i < T * PF_NT; i += (int)blockDim.x) {
            const int t = i / PF_NT, j = i % PF_NT;
            const int tok = S.entry[e0 + t].y * PF_NT + j;
            int rin = -1, ract = 0;
            float sc = 0.f;
            if (tok < m) {
                if (is_shared) { rin = ract = A.n * A.top_k + A.sh_begin + tok; sc = A.scale_s[A.sh_begin + tok]; }
                else { rin = list[tok]; ract = A.g.offset[slot] + tok; sc = A.scale_r[rin]; }
                sc *= A.act_h_scale[rin];
            }
            S.row_in[t][j] = rin;
            S.row_act[t][j] = ract;
            S.scale[t][j] = sc;
        }
        __syncthreads();

        // A B piece holds the activations of TPP token tiles of the run (the last one of an odd run holds one): pieces
        // are numbered i = s * P + p with P = ceil(T / TPP); piece i is the CTA's commit base + i and sits in that
        // commit's buffer.
        const int P = (T + TPP - 1) / TPP, base = committed;
        if constexpr (DownCfg<DT>::TMA_B) {
            // The run's tokens are consecutive rows of act_h (it is written in expert-sorted order), a token tile is
            // one box of the tensor map: 64 rows x 64 halves land in the 128-byte swizzled layout the MMAs read, and the
            // bytes count on the buffer's barrier.  Rows past the expert's last token belong to the next expert (or lie
            // past the array: zeros): their columns of the accumulators are never stored.  A ninth warp issues the copies
            // (the eight working warps meet at a barrier of their own), so that no working thread waits for them.
            const int n_pieces = steps * P;
            const int row0 = (is_shared ? A.n * A.top_k + A.sh_begin : A.g.offset[slot]) + S.entry[e0].y * PF_NT;
            if (warp == DN_THREADS / 32) {
                // the copy warp: piece j goes out as soon as the MMAs that read its buffer (piece j - NB) are done
                for (int j = 0; j < n_pieces && ok; j++) {
                    wait_mma(base + j - NB + 1);
                    if (ok && lane == 0) {
                        const int s_ = j / P, p_ = j % P, buf = (base + j) % NB;
                        const int tp = T - TPP * p_ < TPP ? T - TPP * p_ : TPP;
                        mbar_expect_tx(&S.bar_full[buf], (uint32_t)(tp * PF_NT * DN_KSTEP * 2));
                        for (int t = 0; t < tp; t++)
                            tma_load_2d(b_tile + buf * B_BYTES + t * (PF_NT * DN_KSTEP * 2), &A.act_map, s_ * DN_KSTEP,
                                        row0 + (TPP * p_ + t) * PF_NT, &S.bar_full[buf]);
                    }
                }
                // (a warp that gave up may have copies under way: they land, bounded, before the buffers go)
                if (!ok && lane == 0)
                    for (int g = base; g < base + n_pieces; g++)
                        if (!mbar_wait(&S.bar_full[g % NB], (uint32_t)((g / NB) & 1), 1u << 8)) break;
                committed += n_pieces;
                ph_raw ^= 1;
            } else {
                if (!mbar_wait(&S.bar_raw, ph_raw)) {
                    set_status(A.status, PMOE_ERR_TIMEOUT, 31, e0);
                    ok = false;
                }
                ph_raw ^= 1;
                for (int s = 0; s < steps; s++) {
                    wait_mma(base + s * P);   // the previous step's MMAs still read the A tile
                    tc_fence_after();
                    if (ok) DQ::step(raw + (size_t)r * DQ::ROW_BYTES, s, a_tile, r, part);
                    tc_fence_before();
                    // the working warps meet: the A tile is whole; a thread that gave up takes all of them out together
                    {
                        uint32_t all_ok;
                        asm volatile(
                            "{\n\t.reg .pred p, q;\n\t"
                            "setp.ne.u32 q, %1, 0;\n\t"
                            "barrier.cta.red.and.pred p, 1, %2, q;\n\t"
                            "selp.u32 %0, 1, 0, p;\n\t}"
                            : "=r"(all_ok)
                            : "r"((uint32_t)ok), "n"(DN_THREADS)
                            : "memory");
                        ok = all_ok != 0;
                    }
                    if (!ok) break;
                    if (tid == 0) {
                        fence_proxy_async();   // the A tile's stores went through the generic proxy
                        tc_fence_after();
                        for (int p = 0; p < P && ok; p++) {
                            const int g = base + s * P + p, buf = g % NB;
                            if (!mbar_wait_spin(&S.bar_full[buf], (uint32_t)((g / NB) & 1))) {
                                set_status(A.status, PMOE_ERR_TIMEOUT, 33, g);
                                ok = false;
                                break;
                            }
                            const uint64_t db0 = desc_b0 + (uint64_t)((buf * B_BYTES) >> 4);
                            const int tp = T - TPP * p < TPP ? T - TPP * p : TPP;               // token tiles of this piece
                            const uint32_t idesc = make_idesc(1, 0, 0, PF_NT * tp, PF_M);       // f16 x f16 -> f32, N = 64 tp over its columns
#pragma unroll
                            for (int ks = 0; ks < DN_KSTEP / 16; ks++)   // 16 halves = 32 bytes of K per instruction
                                mma_f16(tmem + 64 * TPP * p, desc_a0 + (uint64_t)(ks * ((2 * PF_M * 16) >> 4)),
                                        db0 + (uint64_t)(ks * (32 >> 4)), idesc, (s > 0 || ks > 0) ? 1u : 0u);
                            tc_commit(&S.bar_b[buf]);
                        }
                    }
                    committed += P;
                }
            }
        } else {
        // The piece travels global -> registers -> shared memory, loaded one piece ahead: eight threads read
        // a token's 128 bytes (a warp reads four whole rows) and store them into one row of the 128-byte swizzled
        // layout, without bank conflicts on either side.  (A cp.async ring two pieces ahead measured the same; its copies cost one
        // shared-memory wavefront per lane where these stores take four per warp.)
        uint4 nb[LPT];
        int ls = 0, lp = 0;   // step and pair of the next piece to load
        auto load_b = [&]() {
#pragma unroll
            for (int j = 0; j < LPT; j++) nb[j] = make_uint4(0, 0, 0, 0);
            if (ls < steps) {
#pragma unroll
                for (int j = 0; j < LPT; j++) {
                    const int tok = tk0 + 32 * j, t = TPP * lp + (tok >> 6);
                    const int rin = t < T ? S.row_in[t][tok & 63] : -1;
                    if (rin >= 0) nb[j] = *reinterpret_cast<const uint4 *>(A.act_h + (size_t)S.row_act[t][tok & 63] * A.F + ls * DN_KSTEP + 8 * chunk);
                }
                if (++lp == P) { lp = 0; ls++; }
            }
        };
        load_b();
        if (!mbar_wait(&S.bar_raw, ph_raw)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 31, e0);
            ok = false;
        }
        ph_raw ^= 1;
        // token tk0 + 32 j: row group (tk0 >> 3) + 4 j, row tk0 & 7 of it, chunk at chunk ^ row
        const uint32_t b_off = (uint32_t)((tk0 >> 3) * 1024 + (tk0 & 7) * 128 + ((chunk ^ (tk0 & 7)) << 4));
        for (int s = 0, i = 0; s < steps && ok; s++) {
            wait_mma(base + i);   // the previous step's MMAs still read the A tile
            tc_fence_after();
            DQ::step(raw + (size_t)r * DQ::ROW_BYTES, s, a_tile, r, part);
            for (int p = 0; p < P && ok; p++, i++) {
                const int buf = (base + i) % NB;
                wait_mma(base + i - NB + 1);   // the MMAs that read this buffer NB pieces ago
                uint8_t *bt = b_tile + buf * B_BYTES + b_off;
#pragma unroll
                for (int j = 0; j < LPT; j++) *reinterpret_cast<uint4 *>(bt + 4096 * j) = nb[j];   // 32 tokens on = four row groups on
                load_b();
                tc_fence_before();
                __syncthreads();
                if (tid == 0) {
                    fence_proxy_async();   // the stores above went through the generic proxy
                    tc_fence_after();
                    // a K slice of 16 halves is two 16-byte chunks further on: the descriptor's address field moves with it
                    const uint64_t db0 = desc_b0 + (uint64_t)((buf * B_BYTES) >> 4);
                    const int tp = T - TPP * p < TPP ? T - TPP * p : TPP;               // token tiles of this piece
                    const uint32_t idesc = make_idesc(1, 0, 0, PF_NT * tp, PF_M);       // f16 x f16 -> f32, N = 64 tp over its columns
#pragma unroll
                    for (int ks = 0; ks < DN_KSTEP / 16; ks++)   // 16 halves = 32 bytes of K per instruction
                        mma_f16(tmem + 64 * TPP * p, desc_a0 + (uint64_t)(ks * ((2 * PF_M * 16) >> 4)),
                                db0 + (uint64_t)(ks * (32 >> 4)), idesc, (s > 0 || ks > 0) ? 1u : 0u);
                    tc_commit(&S.bar_b[buf]);
                }
                committed++;
            }
        }
        }
        wait_mma(committed);
        tc_fence_after();
        if (ok && warp < DN_THREADS / 32) {
            // row (32 * (warp & 3) + lane) of the block: a warp reaches the 32 lanes of its quarter; the two warps
            // of a quarter split the run's tiles
            const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
            const int row = h0 + (warp & 3) * 32 + lane;
            for (int t = warp >> 2; t < T; t += 2) {
#pragma unroll
                for (int cc = 0; cc < PF_NT / 16; cc++) {
                    uint32_t v[16];
                    tmem_ld16(lane_addr + 64 * t + cc * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int rout = S.row_in[t][cc * 16 + j];
                        if (rout >= 0) A.partial[(size_t)rout * A.H + row] = __uint_as_float(v[j]) * S.scale[t][cc * 16 + j];
                    }
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);   // accumulators, tiles and tables are free for the next run; a failure ends the CTA as one
        tc_fence_after();
        e0 = e1;
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, DN_COLS);
}

// Quantisation of an activated row the way the row's down matrix wants it (Q8_K for K-quants, Q8_0 for Q8_0:
// BlockQ8K / BlockQ8_0::from_float, bit-exact), written back as fp16 d*q for the fp16 down GEMM
// A row whose largest magnitude would leave the fp16 range is written times a power of two 2^-e (exact), and
// row_scale[r] = 2^e goes back in when the down GEMM's accumulators are drained; other rows have scale 1.
__global__ void __launch_bounds__(64) k_act_fakequant_h(const float *__restrict__ act, int F, int n_routed_rows,
                                                        const int *__restrict__ sorted_pairs, const int *__restrict__ n_sorted,
                                                        bool routed, bool kq_routed, bool kq_shared,
                                                        __half *__restrict__ out, float *__restrict__ row_scale)
{
    __shared__ float s_amax[2];
    // CTA w < n_routed_rows writes row w of the output: the w-th pair in expert-sorted order (the down GEMM fetches
    // an expert's token tiles as boxes of consecutive rows); the shared expert's rows keep their places
    const int w = blockIdx.x;
    if (w < n_routed_rows && (!routed || w >= *n_sorted)) return;
    const int r = w < n_routed_rows ? sorted_pairs[w] : w;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool kq = r < n_routed_rows ? kq_routed : kq_shared;
    float down = 1.f;   // 2^-e
    {
        float am = 0.f;
        for (int i = threadIdx.x; i < F; i += 64) am = fmaxf(am, fabsf(act[(size_t)r * F + i]));
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, s));
        if (lane == 0) s_amax[warp] = am;
        __syncthreads();
        am = fmaxf(s_amax[0], s_amax[1]);
        // quantised values stay below 1.01 * amax; keep them under 32768
        float up = 1.f;
        while (am * down > 32768.f) { down *= 0.5f; up *= 2.f; }
        if (threadIdx.x == 0) row_scale[r] = up;
    }
    if (!kq) {
        // Q8_0: blocks of 32, d = amax / 127 kept as f16, q = round_half_away(x * (1 / d))
        for (int b = warp; b < F / QK8_0; b += 2) {
            const float x = act[(size_t)r * F + b * QK8_0 + lane];
            float amax = fabsf(x);
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            const float d = __fdiv_rn(amax, 127.f);
            const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
            const float q = roundf(__fmul_rn(x, id));
            const float df = __half2float(__float2half_rn(d));
            out[(size_t)w * F + b * QK8_0 + lane] = __float2half_rn((q * df) * down);
        }
        return;
    }
    for (int b = warp; b < F / QK_K; b += 2) {
        const float *src = act + (size_t)r * F + b * QK_K;
        float v[8];
        const float4 a = reinterpret_cast<const float4 *>(src)[2 * lane], c = reinterpret_cast<const float4 *>(src)[2 * lane + 1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        float amax = 0.f, mx = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (amax < fabsf(v[j])) { amax = fabsf(v[j]); mx = v[j]; }
        int who = lane;
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, amax, s), om = __shfl_xor_sync(0xffffffffu, mx, s);
            const int ow = __shfl_xor_sync(0xffffffffu, who, s);
            if (oa > amax || (oa == amax && ow < who)) { amax = oa; mx = om; who = ow; }
        }
        uint4 o = make_uint4(0, 0, 0, 0);
        if (amax != 0.f) {
            const float iscale = __fdiv_rn(-128.f, mx), d = __fdiv_rn(1.f, iscale);
            __half2 h[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float q0 = fminf(roundf(__fmul_rn(iscale, v[2 * j])), 127.f);
                const float q1 = fminf(roundf(__fmul_rn(iscale, v[2 * j + 1])), 127.f);
                h[j] = __floats2half2_rn((q0 * d) * down, (q1 * d) * down);
            }
            o = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                           *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
        }
        *reinterpret_cast<uint4 *>(out + (size_t)w * F + b * QK_K + 8 * lane) = o;
    }
}

// number of token tiles a call can need at most: sum_e ceil(m_e / NT) <= pairs / NT + active experts
static int max_routed_tiles(const LayerDev &L, int n, int top_k)
{
    long pairs = (long)n * top_k;
    long act = pairs < L.E_local ? pairs : L.E_local;
    return (int)(pairs / PF_NT + act);
}

static bool rows_map(const uint8_t *w, size_t rows, size_t row_bytes, uint32_t box_bytes, CUtensorMap *out);

static size_t row_bytes_of_gate(const LayerDev &L, int dt) { return row_bytes(dt, L.H); }

static bool pf_gu_ok(int dt) { return dt == PMOE_Q4_K || dt == PMOE_Q8_0; }
static bool pf_dn_ok(int dt) { return dt == PMOE_Q6_K || dt == PMOE_Q4_K || dt == PMOE_Q8_0; }

bool prefill_supported(const LayerDev &L, const Workspace &ws, bool routed, bool shared)
{
    if (L.H != 2048 || L.F != 512) return false;
    // the Q4_K kernel gathers the quantised rows through a tensor map made for the workspace's own array
    if (((routed && L.gate_dtype == PMOE_Q4_K) || (shared && L.sh_gate_dtype == PMOE_Q4_K)) &&
        !(ws.xq_map_ok && ws.xq_map_base == ws.x_q8k.qs))
        return false;
    if (((routed && L.gate_dtype == PMOE_Q8_0) || (shared && L.sh_gate_dtype == PMOE_Q8_0)) &&
        !(ws.xq80_map_ok && ws.xq80_map_base == ws.x_q80.qs && ws.xd80_map_base == ws.x_q80.d))
        return false;
    if (routed && !pf_gu_ok(L.gate_dtype)) return false;
    if (shared && !pf_gu_ok(L.sh_gate_dtype)) return false;
    return true;
}

cudaError_t launch_gate_up_prefill(const LayerDev &L, const Workspace &ws, int n, int top_k, bool routed, bool shared,
                                   cudaStream_t s)
{
    if (routed && shared && L.gate_dtype != L.sh_gate_dtype) {   // two types: one launch each
        cudaError_t e = launch_gate_up_prefill(L, ws, n, top_k, true, false, s);
        if (e != cudaSuccess) return e;
        return launch_gate_up_prefill(L, ws, n, top_k, false, true, s);
    }
    const int dt = routed ? L.gate_dtype : L.sh_gate_dtype;
    GuArgs A{};
    A.gate = L.gate_exps; A.up = L.up_exps;
    A.expert_bytes = row_bytes(L.gate_dtype, L.H) * L.F;
    A.sgate = L.sh_gate; A.sup = L.sh_up;
    A.has_shared = shared; A.routed = routed;
    A.n = n; A.top_k = top_k; A.H = L.H; A.F = L.F;
    A.sh_begin = ws.sh_begin; A.sh_count = ws.sh_count;
    A.g = ws.groups;
    A.tile_prefix = ws.groups.tile_prefix;
    A.xq = dt == PMOE_Q8_0 ? ws.x_q80 : ws.x_q8k;
    {
        const bool q80 = dt == PMOE_Q8_0;
        memcpy(&A.xq_map, q80 ? ws.xq80_map : ws.xq_map, sizeof(CUtensorMap));
        memcpy(&A.xd_map, ws.xd80_map, sizeof(CUtensorMap));
        const size_t row_bytes = row_bytes_of_gate(L, dt);
        const uint32_t box = q80 ? 8 * Q8_0_BYTES : Q4_K_BYTES;
        bool got = true;
        if (routed) got = rows_map(L.gate_exps, (size_t)L.E_local * L.F, row_bytes, box, &A.w_map[0]) &&
                          rows_map(L.up_exps, (size_t)L.E_local * L.F, row_bytes, box, &A.w_map[1]);
        if (got && shared) got = rows_map(L.sh_gate, (size_t)L.F, row_bytes, box, &A.w_map[2]) && rows_map(L.sh_up, (size_t)L.F, row_bytes, box, &A.w_map[3]);
        if (!got) return cudaErrorInvalidValue;
    }
    A.act = ws.act;
    A.status = ws.status;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_gu_prefill, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(GuSmem) + 1024 + 128);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(k_gu_prefill_q80, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Gu80Smem) + 1024 + 128);

        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int tiles = (routed ? max_routed_tiles(L, n, top_k) : 0) + (shared ? (ws.sh_count + PF_NT - 1) / PF_NT : 0);
    dim3 grid(L.F / 64, tiles);
    if (dt == PMOE_Q8_0) k_gu_prefill_q80<<<grid, GU_THREADS, sizeof(Gu80Smem) + 1024 + 128, s>>>(A);
    else k_gu_prefill<<<dim3(L.F / 64, (tiles + GU_REPS - 1) / GU_REPS), GU_THREADS, sizeof(GuSmem) + 1024 + 128, s>>>(A);
    count_launch();
    return cudaGetLastError();
}

using TmaEncode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmaEncode tma_encoder()
{
    static TmaEncode encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && fn &&
            q == cudaDriverEntryPointSuccess)
            encode = (TmaEncode)fn;
    }
    return encode;
}

// row-major [rows, cols] of `elem_bytes`-byte elements, boxes of box_rows x box_cols; 128-byte swizzle (box rows of 128
// bytes) or none (box rows a multiple of 16 bytes)
static bool encode_2d(void *out_map, CUtensorMapDataType dt, size_t elem_bytes, const void *base, size_t rows, size_t cols,
                      uint32_t box_cols, uint32_t box_rows, bool swizzle = true)
{
    TmaEncode encode = tma_encoder();
    if (!encode || rows == 0 || cols % box_cols != 0 || ((uintptr_t)base & 15) || (cols * elem_bytes) % 16 != 0) return false;
    if (swizzle ? box_cols * elem_bytes != 128 : (box_cols * elem_bytes) % 16 != 0) return false;
    CUtensorMap m;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(cols * elem_bytes)};
    const cuuint32_t box[2] = {box_cols, box_rows}, estr[2] = {1, 1};
    if (encode(&m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(out_map, &m, sizeof(m));
    return true;
}

bool make_act_h_map(Workspace &ws, size_t rows, int F)
{
    return encode_2d(ws.act_h_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ws.act_h, rows, (size_t)F, DN_KSTEP, PF_NT);
}

// Descriptor of a quantised matrix [rows, row_bytes / 4] as 4-byte words, boxes of 64 rows x box_bytes.  The matrices are static
// (a call with block multipliers installed brings other arrays): the descriptors are kept by array and shape.
static bool rows_map(const uint8_t *w, size_t rows, size_t row_bytes, uint32_t box_bytes, CUtensorMap *out)
{
    struct Key {
        const uint8_t *w;
        size_t rows, row_bytes;
        uint32_t box;
        bool operator<(const Key &o) const
        {
            if (w != o.w) return w < o.w;
            if (rows != o.rows) return rows < o.rows;
            if (row_bytes != o.row_bytes) return row_bytes < o.row_bytes;
            return box < o.box;
        }
    };
    static std::mutex mu;
    static std::map<Key, CUtensorMap> cache;
    std::lock_guard<std::mutex> lock(mu);
    const Key key{w, rows, row_bytes, box_bytes};
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        // (as 4-byte words: a box dimension may not exceed 256 elements, and eight Q8_0 blocks are 272 bytes)
        if (row_bytes % 4 != 0 || box_bytes % 4 != 0 ||
            !encode_2d(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, w, rows, row_bytes / 4, box_bytes / 4, 64, false))
            return false;
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

bool make_xq_map(Workspace &ws, size_t rows, int H)
{
    ws.xq_map_base = ws.x_q8k.qs;
    ws.xq80_map_base = ws.x_q80.qs;
    ws.xd80_map_base = ws.x_q80.d;
    ws.xq80_map_ok = encode_2d(ws.xq80_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ws.x_q80.qs, rows, (size_t)H, 128, 1) &&
                     encode_2d(ws.xd80_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ws.x_q80.d, rows, (size_t)H / QK8_0, 4, 1, false);
    return encode_2d(ws.xq_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ws.x_q8k.qs, rows, (size_t)H, 128, 1);
}

bool prefill_down_supported(const LayerDev &L, const Workspace &ws, bool routed, bool shared)
{
    if (L.H != 2048 || L.F != 512) return false;
    if (!ws.act_h_map_ok) return false;
    if (routed && !pf_dn_ok(L.down_dtype)) return false;
    if (shared && !pf_dn_ok(L.sh_down_dtype)) return false;
    return true;
}

template <int DT>
static cudaError_t launch_down_t(const DownArgs &A, dim3 grid, cudaStream_t s)
{
    constexpr size_t smem = PF_M * DN_KSTEP * 2 + DownCfg<DT>::NB * DownCfg<DT>::PT * DN_KSTEP * 2 +
                            ((PF_M * DownDequant<DT>::ROW_BYTES + 127) / 128) * 128 + sizeof(DownSmemHdr) + 128 + 1024;
    static_assert(smem <= 115712, "two CTAs of the down GEMM share an SM");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_down_prefill<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    k_down_prefill<DT><<<grid, DownCfg<DT>::THREADS, smem, s>>>(A);
    count_launch();
    return cudaGetLastError();
}

static cudaError_t launch_down_gemm(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k, bool routed,
                                    bool shared, cudaStream_t s)
{
    DownArgs A{};
    A.down = L.down_exps;
    A.expert_bytes = row_bytes(L.down_dtype, L.F) * L.H;
    A.sdown = L.sh_down;
    A.has_shared = shared; A.routed = routed;
    A.n = n; A.top_k = top_k; A.H = L.H; A.F = L.F;
    A.sh_begin = ws.sh_begin; A.sh_count = ws.sh_count;
    A.g = ws.groups;
    A.tile_prefix = ws.groups.tile_prefix;
    A.act_h = ws.act_h;
    static_assert(sizeof(CUtensorMap) == sizeof(ws.act_h_map), "the workspace holds the descriptor as bytes");
    memcpy(&A.act_map, ws.act_h_map, sizeof(CUtensorMap));
    A.act_h_scale = ws.act_h_scale;
    A.scale_r = w;
    A.scale_s = ws.sh_sigmoid;
    A.partial = ws.partial;
    A.status = ws.status;
    const int tiles = (routed ? max_routed_tiles(L, n, top_k) : 0) + (shared ? (ws.sh_count + PF_NT - 1) / PF_NT : 0);
    dim3 grid(L.H / PF_M, (tiles + DN_TILES - 1) / DN_TILES);
    const int dt = routed ? L.down_dtype : L.sh_down_dtype;
    if (dt == PMOE_Q6_K) return launch_down_t<PMOE_Q6_K>(A, grid, s);
    if (dt == PMOE_Q8_0) return launch_down_t<PMOE_Q8_0>(A, grid, s);
    return launch_down_t<PMOE_Q4_K>(A, grid, s);
}

cudaError_t launch_down_prefill(const LayerDev &L, const Workspace &ws, const float *w, int n, int top_k, bool routed,
                                bool shared, cudaStream_t s)
{
    const int rows = n * top_k + (shared ? n : 0);
    k_act_fakequant_h<<<rows, 64, 0, s>>>(ws.act, L.F, n * top_k, ws.groups.pairs, ws.groups.offset + L.E_local, routed,
                                          is_kquant(L.down_dtype), is_kquant(L.sh_down_dtype), ws.act_h, ws.act_h_scale);
    count_launch();
    if (routed && shared && L.down_dtype != L.sh_down_dtype) {   // two types: one launch each
        cudaError_t e = launch_down_gemm(L, ws, w, n, top_k, true, false, s);
        if (e != cudaSuccess) return e;
        return launch_down_gemm(L, ws, w, n, top_k, false, true, s);
    }
    return launch_down_gemm(L, ws, w, n, top_k, routed, shared, s);
}

}  // namespace pmoe
