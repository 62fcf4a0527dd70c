// Tensor-core (mma.sync) kernels of the decode path: expert-grouped GEMV-sized products where a
// handful of tokens share an expert, over raw GGUF blocks streamed through the shared-memory ring.
#include "pmoe_gemv.cuh"

namespace pmoe {

// ---------------------------------------------------------------- Q4_K gate/up on the tensor cores
// The same gate/up step for Q4_K routed experts with the dot products on the tensor cores
// (mma.sync.m16n8k32, u8 weights x s8 activations -> s32): sixteen weight rows are the M side, up to
// eight tokens of the expert the N side, and one 32-weight sub-block -- the span of one 6-bit
// scale -- the K of one instruction, so the integer sub-block sums are exact and meet their scales
// as integers exactly like the dp4a path.  One instruction replaces 16 x tokens dp4a, and no
// shuffle reduction over the reduction dimension is left.
//
// An item is still 16 gate + 16 up rows of one expert, but a slot with more than eight tokens is
// walked once per group of eight (the ring delivers its items again, from L2).  Warp w of the eight
// compute warps owns block column w of all 32 rows (K = 2048 = 8 blocks), so the eight tokens'
// quantised activations of that column stay in 16 registers per lane for the whole expert.  The
// mins term sum_j m_j * bsum_j goes through two more instructions over the partial sums split into
// signed byte digits (bsum = 64 h + l).  The eight warps' partial sums meet in shared memory, in
// the part of the ring slot the warp itself has finished reading, and are added in warp order.
//
// An item arrives as eight bulk copies of four consecutive rows (4608 bytes); the quads of a matrix sit
// 4640 bytes apart, so that with one row of every quad on the row positions of a half-warp's fragment
// the 8-byte loads fall into 32 different banks (rows 1152 bytes apart would all meet in the same ones).
constexpr int Q4K_ROW = 8 * Q4_K_BYTES;                 // 1152: one row of K = 2048
constexpr int Q4K_QUAD = 4 * Q4K_ROW + 32;              // 4640: four consecutive rows (one bulk copy) and 32 bytes of padding
constexpr int Q4K_TILE = 4 * Q4K_QUAD;                  // 18 560: the 16 rows of one matrix
constexpr int MMA_STAGE_BYTES = 37376;                  // 2 x 18 560 rounded up to a multiple of 128
static_assert(MMA_STAGE_BYTES % 128 == 0 && MMA_STAGE_BYTES >= STAGE_BYTES && MMA_STAGE_BYTES >= 2 * Q4K_TILE,
              "ring slot of the tensor-core GEMV");
// byte offset of row r (0..15) of a matrix inside its tile
__device__ inline int q4k_row_off(int r) { return (r >> 2) * Q4K_QUAD + (r & 3) * Q4K_ROW; }

__device__ inline void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                    uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Items of the tensor-core kernel, in order: (slot, token group, chunk), chunk fastest.  Every item
// costs the same, so a CTA takes an equal share of the item count.
struct MmaCursor {
    int slot, group, chunk, groups;   // groups = token groups of `slot`
};

struct MmaWork {
    int n_active, cpe, groups_sh;   // groups_sh = 0 when the shared expert is not served by these items
    const int *prefix;              // [n_active + 1] exclusive prefix of ceil(count / 8) over the active slots (global)

    __device__ inline int routed_groups() const { return n_active ? prefix[n_active] : 0; }
    __device__ inline long total() const { return (long)cpe * (routed_groups() + groups_sh); }
    __device__ inline MmaCursor at(long q) const
    {
        const int G = (int)(q / cpe), chunk = (int)(q % cpe);
        const int rg = routed_groups();
        if (G >= rg) return MmaCursor{n_active, G - rg, chunk, groups_sh};
        int lo = 0, hi = n_active - 1;   // largest slot with prefix[slot] <= G
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= G) lo = mid; else hi = mid - 1;
        }
        return MmaCursor{lo, G - prefix[lo], chunk, prefix[lo + 1] - prefix[lo]};
    }
    __device__ inline void advance(MmaCursor &c) const
    {
        if (++c.chunk < cpe) return;
        c.chunk = 0;
        if (++c.group < c.groups) return;
        c.group = 0;
        c.slot++;
        c.groups = c.slot < n_active ? prefix[c.slot + 1] - prefix[c.slot] : groups_sh;
    }
};

// The CTA's share of the items: its first item and its item count, found by all threads together.  Every thread
// fetches the prefix entries of its candidate slots before anything depends on them, so the search costs two
// round trips to memory (the number of active slots, then the total) instead of a binary search's chain of them.
__device__ inline void mma_plan(MmaWork &work, const GemvArgs &A, MmaCursor *s_first, int *s_items)
{
    constexpr int CAND = 4;   // candidate slots per thread: covers E_local <= 4 * 288
    int lo[CAND], hi[CAND];
#pragma unroll
    for (int i = 0; i < CAND; i++) {
        const int sl = threadIdx.x + i * blockDim.x;
        lo[i] = hi[i] = 0;
        if (sl < A.e_local) { lo[i] = work.prefix[sl]; hi[i] = work.prefix[sl + 1]; }
    }
    work.n_active = A.routed ? *A.g.n_active : 0;
    const long total = work.total();
    const long q0 = total * blockIdx.x / gridDim.x, q1 = total * (blockIdx.x + 1) / gridDim.x;
    if (threadIdx.x == 0) *s_items = (int)(q1 - q0);
    if (q1 <= q0) {
        if (threadIdx.x == 0) *s_first = MmaCursor{0, 0, 0, 0};
        return;
    }
    const int G = (int)(q0 / work.cpe), chunk = (int)(q0 % work.cpe);
    const int rg = work.routed_groups();
    if (G >= rg) {
        if (threadIdx.x == 0) *s_first = MmaCursor{work.n_active, G - rg, chunk, work.groups_sh};
        return;
    }
#pragma unroll
    for (int i = 0; i < CAND; i++) {
        const int sl = threadIdx.x + i * blockDim.x;
        if (sl < work.n_active && lo[i] <= G && G < hi[i]) *s_first = MmaCursor{sl, G - lo[i], chunk, hi[i] - lo[i]};
    }
}

struct Q4Hdr {
    float d16, dmin;              // d / 16 (high nibbles stay in place) and dmin
    uint32_t sca, scb, mna, mnb;  // 6-bit scales 0..3 / 4..7 and mins 0..3 / 4..7 as bytes
};

__device__ inline Q4Hdr q4k_hdr(const uint4 h)
{
    Q4Hdr o;
    o.d16 = half_bits_to_float((uint16_t)(h.x & 0xffffu)) * 0.0625f;
    o.dmin = half_bits_to_float((uint16_t)(h.x >> 16));
    o.sca = h.y & 0x3F3F3F3Fu;
    o.mna = h.z & 0x3F3F3F3Fu;
    o.scb = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    o.mnb = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    return o;
}

// The lists of the token group that follows the current one, fetched one dependent load per item while the
// current group's items are computed (a warp issues in order: a chain of dependent loads would stall it for
// the whole chain, and under the weight stream a single access to L2 or HBM already takes microseconds).
struct LookAhead {
    int slot, group, step, e, m, off, row;   // row: pair id of token (lane & 7) of that group, -1 if none
    __device__ inline void start(const MmaCursor &cur)
    {
        slot = cur.slot; group = cur.group + 1;
        if (group >= cur.groups) { slot++; group = 0; }
        step = 0; row = -1; m = 0; e = 0; off = 0;
    }
    __device__ inline void advance(const GemvArgs &A, const MmaWork &work, int lane)
    {
        if (slot >= work.n_active || step > 2) return;   // the shared expert (or nothing) follows: no lists to read
        if (step == 0) {
            e = A.g.active[slot];
        } else if (step == 1) {
            m = A.g.count[e];
            off = A.g.offset[e];
        } else {
            const int i = GEMV_TG_MMA * group + (lane & 7);
            row = i < m ? A.g.pairs[off + i] : -1;
        }
        step++;
    }
    __device__ inline bool ready(const MmaWork &work, int s, int g) const
    {
        return s == slot && g == group && s < work.n_active && step > 2;
    }
};

__device__ inline void mma_u8s8_k32_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Sums of the quants under the four sub-blocks 4t .. 4t+3 (pairs of the Q8_K partial sums of 16) as four bytes:
// their high digits (v >> 6) or low digits (v & 63), v = 64 h + l.
__device__ inline uint32_t q4_bsum_digits(uint4 bs, bool low)
{
    const uint32_t w4[4] = {bs.x, bs.y, bs.z, bs.w};
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int v = (int)(int16_t)(w4[i] & 0xffffu) + (int)(int16_t)(w4[i] >> 16);
        o |= (uint32_t)((low ? (v & 63) : (v >> 6)) & 0xFF) << (8 * i);
    }
    return o;
}

// How many tokens a group is laid out for decides what the eight accumulator columns mean:
//   TP 2: (sub-block slot 0..3) x (token 0..1) -- the four even sub-blocks of a block share one accumulator (a token's
//         activations are non-zero only in the columns of the slot the instruction covers), the four odd ones another;
//   TP 4: (slot 0..1) x (token 0..3), two accumulators per parity;
//   TP 8: the columns are the tokens, one accumulator per sub-block.
// Fewer accumulators mean fewer integer multiplies by the 6-bit scales afterwards.
template <int TP> struct GuGroup {
    static constexpr int NF = TP == 2 ? 1 : 2;   // tokens of the lane's final values
    uint32_t bq[8][2];   // B operand per sub-block of block column `warp` (zero where the lane's column belongs to another slot)
    uint32_t bm[2];      // partial-sum digits for the mins products (TP 2: one register, the digit follows the column)
    float dx[NF];        // activation scale of the lane's final tokens in this block column
    int r_orow, r_row;   // cross-warp sum: output row and row inside the item of the value this thread finishes (-1: none)
};

// my_row = pair id of token (lane & 7) of the group (routed experts).  Called by all lanes; shuffles come first.
template <int TP>
__device__ inline void gu_load_group(const GemvArgs &A, bool is_sh, int my_row, int t0, int cnt, int warp, int lane, GuGroup<TP> &G)
{
    const int g = lane >> 2, t = lane & 3;
    const QAct &in = is_sh ? A.in_s : A.in_r;
    const int my_act = my_row >= 0 ? my_row / A.top_k : 0;
    auto act_row = [&](int i) -> size_t {   // row of the quantised input of token i
        const int r = __shfl_sync(0xffffffffu, my_act, i & 7);
        return is_sh ? (size_t)(A.sh_begin + t0 + i) : (size_t)r;
    };
    const int tok_b = TP == 2 ? (g & 1) : TP == 4 ? (g & 3) : g;
    const int tok_m = TP == 2 ? ((g >> 1) & 1) : tok_b;
    const size_t row_b = act_row(tok_b), row_m = act_row(tok_m);
    size_t row_f[GuGroup<TP>::NF];
    int tok_f[GuGroup<TP>::NF];
#pragma unroll
    for (int j = 0; j < GuGroup<TP>::NF; j++) {
        tok_f[j] = TP == 2 ? (t & 1) : TP == 4 ? 2 * (t & 1) + j : 2 * t + j;
        row_f[j] = act_row(tok_f[j]);
    }
    // the value this thread finishes in the cross-warp sum: (row r_row of the item, token r_tok)
    constexpr int TPV = 8 / TP;   // threads per value
    const int vi = warp * (16 / TPV) + (lane & 15) / TPV;
    const int r_tok = vi % TP;
    const int r_pair = __shfl_sync(0xffffffffu, my_row, r_tok & 7);
    G.r_row = vi / TP;
    G.r_orow = r_tok < cnt ? (is_sh ? A.n * A.top_k + A.sh_begin + t0 + r_tok : r_pair) : -1;

#pragma unroll
    for (int j = 0; j < 8; j++) G.bq[j][0] = G.bq[j][1] = 0;
    if (tok_b < cnt) {
        const int8_t *xp = in.qs + row_b * 2048 + 256 * warp + 8 * t;
        if (TP == 2) {          // the lane's column belongs to slot g >> 1 = chunk c: sub-blocks 2c (low nibbles), 2c + 1
            const int c_own = g >> 1;
            const uint2 lo = *reinterpret_cast<const uint2 *>(xp + 64 * c_own);
            const uint2 hi = *reinterpret_cast<const uint2 *>(xp + 64 * c_own + 32);
#pragma unroll
            for (int c = 0; c < 4; c++)
                if (c == c_own) { G.bq[2 * c][0] = lo.x; G.bq[2 * c][1] = lo.y; G.bq[2 * c + 1][0] = hi.x; G.bq[2 * c + 1][1] = hi.y; }
        } else if (TP == 4) {   // slot g >> 2: chunks c with (c & 1) == slot
            const int s_own = g >> 2;
#pragma unroll
            for (int a = 0; a < 2; a++) {
                const uint2 lo = *reinterpret_cast<const uint2 *>(xp + 64 * (2 * a + s_own));
                const uint2 hi = *reinterpret_cast<const uint2 *>(xp + 64 * (2 * a + s_own) + 32);
#pragma unroll
                for (int sl = 0; sl < 2; sl++)
                    if (sl == s_own) {
                        G.bq[2 * (2 * a + sl)][0] = lo.x; G.bq[2 * (2 * a + sl)][1] = lo.y;
                        G.bq[2 * (2 * a + sl) + 1][0] = hi.x; G.bq[2 * (2 * a + sl) + 1][1] = hi.y;
                    }
            }
        } else {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint2 lo = *reinterpret_cast<const uint2 *>(xp + 64 * c);
                const uint2 hi = *reinterpret_cast<const uint2 *>(xp + 64 * c + 32);
                G.bq[2 * c][0] = lo.x; G.bq[2 * c][1] = lo.y;
                G.bq[2 * c + 1][0] = hi.x; G.bq[2 * c + 1][1] = hi.y;
            }
        }
    }
    // mins products: K positions 0..7 carry the eight sub-block sums; lanes t = 0, 1 hold them
    G.bm[0] = G.bm[1] = 0;
    if (t < 2 && tok_m < cnt) {
        const uint4 bs = *reinterpret_cast<const uint4 *>(in.bsums + row_m * 128 + 16 * warp + 8 * t);
        if (TP == 2) {
            G.bm[0] = q4_bsum_digits(bs, (g & 1) != 0);   // column g = (.., token (g>>1)&1, digit g&1)
        } else {
            G.bm[0] = q4_bsum_digits(bs, false);
            G.bm[1] = q4_bsum_digits(bs, true);
        }
    }
#pragma unroll
    for (int j = 0; j < GuGroup<TP>::NF; j++) G.dx[j] = tok_f[j] < cnt ? in.d[row_f[j] * 8 + warp] : 0.f;
}

// One item (16 gate + 16 up rows in `stage`) against the group: this warp's block column, then the sum over the
// eight warps in shared memory, silu(gate) * up and the store.
template <int TP>
__device__ inline void gu_item(const GemvArgs &A, uint8_t *stage, const GuGroup<TP> &G, int chunk, bool compute, int warp,
                               int lane)
{
    const int g = lane >> 2, t = lane & 3;
    // tile rows under fragment rows g and g + 8: a half-warp (g = 0..3 or 4..7) meets one row of every quad, whose
    // starts are 32 bytes apart modulo 128, so its 8-byte loads fall into 32 different banks
    const int ra = 4 * (g & 3) + (g >> 2), rb = ra + 2;
    constexpr int NV = TP == 2 ? 1 : TP == 4 ? 2 : 4;
    float acc[2][NV];
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
#pragma unroll
        for (int i = 0; i < NV; i++) acc[mt][i] = 0.f;
        if (!compute) continue;
        const uint8_t *p0 = stage + mt * Q4K_TILE + q4k_row_off(ra) + Q4_K_BYTES * warp;
        const uint8_t *p1 = p0 + 2 * Q4K_ROW;
        const uint4 h0 = *reinterpret_cast<const uint4 *>(p0);
        const uint4 h1 = *reinterpret_cast<const uint4 *>(p1);
        // mins of both rows as the A operand of the mins products: lane t = 0 carries m_0..3, t = 1 m_4..7
        const uint32_t am0 = t == 0 ? (h0.z & 0x3F3F3F3Fu) : t == 1 ? (((h0.w >> 4) & 0x0F0F0F0Fu) | ((h0.z >> 2) & 0x30303030u)) : 0u;
        const uint32_t am1 = t == 0 ? (h1.z & 0x3F3F3F3Fu) : t == 1 ? (((h1.w >> 4) & 0x0F0F0F0Fu) | ((h1.z >> 2) & 0x30303030u)) : 0u;
        if (TP == 8) {
            const Q4Hdr k0 = q4k_hdr(h0), k1 = q4k_hdr(h1);
            int ie[4] = {0, 0, 0, 0}, io[4] = {0, 0, 0, 0};   // even (low-nibble) and odd (high-nibble, x16) sub-blocks
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(p0 + 16 + 32 * c + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(p1 + 16 + 32 * c + 8 * t);
                const uint32_t sw0 = c < 2 ? k0.sca : k0.scb, sw1 = c < 2 ? k1.sca : k1.scb;
                int cc[4];
                mma_u8s8_k32(cc, q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, G.bq[2 * c][0],
                             G.bq[2 * c][1]);
                {
                    const int s0 = (int)__byte_perm(sw0, 0u, 0x4440u + 2 * (c & 1)), s1 = (int)__byte_perm(sw1, 0u, 0x4440u + 2 * (c & 1));
                    ie[0] += cc[0] * s0; ie[1] += cc[1] * s0; ie[2] += cc[2] * s1; ie[3] += cc[3] * s1;
                }
                mma_u8s8_k32(cc, q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u,
                             G.bq[2 * c + 1][0], G.bq[2 * c + 1][1]);
                {
                    const int s0 = (int)__byte_perm(sw0, 0u, 0x4441u + 2 * (c & 1)), s1 = (int)__byte_perm(sw1, 0u, 0x4441u + 2 * (c & 1));
                    io[0] += cc[0] * s0; io[1] += cc[1] * s0; io[2] += cc[2] * s1; io[3] += cc[3] * s1;
                }
            }
            int ch[4], cl[4];
            mma_u8s8_k32(ch, am0, am1, 0u, 0u, G.bm[0], 0u);
            mma_u8s8_k32(cl, am0, am1, 0u, 0u, G.bm[1], 0u);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const Q4Hdr &k = i < 2 ? k0 : k1;
                acc[mt][i] = G.dx[i & 1] * (k.d16 * (float)(16 * ie[i] + io[i]) - k.dmin * (float)(64 * ch[i] + cl[i]));
            }
        } else {
            // accumulators: TP 2: [0] even, [1] odd sub-blocks; TP 4: [2a + parity] for chunks 2a, 2a + 1
            constexpr int NA = TP == 2 ? 2 : 4;
            int cs[NA][4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint2 q0 = *reinterpret_cast<const uint2 *>(p0 + 16 + 32 * c + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2 *>(p1 + 16 + 32 * c + 8 * t);
                const int ae = TP == 2 ? 0 : 2 * (c >> 1), ao = ae + 1;
                const bool first = TP == 2 ? c == 0 : (c & 1) == 0;
                if (first) {
                    mma_u8s8_k32(cs[ae], q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu,
                                 G.bq[2 * c][0], G.bq[2 * c][1]);
                    mma_u8s8_k32(cs[ao], q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u,
                                 G.bq[2 * c + 1][0], G.bq[2 * c + 1][1]);
                } else {
                    mma_u8s8_k32_acc(cs[ae], q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu,
                                     G.bq[2 * c][0], G.bq[2 * c][1]);
                    mma_u8s8_k32_acc(cs[ao], q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u,
                                     G.bq[2 * c + 1][0], G.bq[2 * c + 1][1]);
                }
            }
            // the lane's columns 2t, 2t+1 belong to one slot: TP 2: chunk t; TP 4: chunk t >> 1 (first pair), 2 + (t >> 1)
            int v[4];
            if (TP == 2) {
                // scales of sub-blocks 2t, 2t+1 as a byte pair, without a branch
                const uint32_t sh = 16 * (t & 1);
                const uint32_t y0 = h0.y >> sh, y1 = h1.y >> sh;
                const uint32_t lo0 = y0 & 0x3F3Fu, lo1 = y1 & 0x3F3Fu;
                const uint32_t hi0 = ((h0.w >> sh) & 0x0F0Fu) | ((y0 >> 2) & 0x3030u), hi1 = ((h1.w >> sh) & 0x0F0Fu) | ((y1 >> 2) & 0x3030u);
                const uint32_t sp0 = t < 2 ? lo0 : hi0, sp1 = t < 2 ? lo1 : hi1;
                const int se0 = (int)(sp0 & 0xFFu) << 4, so0 = (int)(sp0 >> 8), se1 = (int)(sp1 & 0xFFu) << 4, so1 = (int)(sp1 >> 8);
                v[0] = se0 * cs[0][0] + so0 * cs[1][0];
                v[1] = se0 * cs[0][1] + so0 * cs[1][1];
                v[2] = se1 * cs[0][2] + so1 * cs[1][2];
                v[3] = se1 * cs[0][3] + so1 * cs[1][3];
            } else {
                const uint32_t sh = 16 * (t >> 1);
                const uint32_t y0 = h0.y >> sh, y1 = h1.y >> sh;
                const uint32_t a0 = y0 & 0x3F3Fu, a1 = y1 & 0x3F3Fu;   // chunk t >> 1
                const uint32_t b0 = ((h0.w >> sh) & 0x0F0Fu) | ((y0 >> 2) & 0x3030u), b1 = ((h1.w >> sh) & 0x0F0Fu) | ((y1 >> 2) & 0x3030u);
                const int ae0 = (int)(a0 & 0xFFu) << 4, ao0 = (int)(a0 >> 8), ae1 = (int)(a1 & 0xFFu) << 4, ao1 = (int)(a1 >> 8);
                const int be0 = (int)(b0 & 0xFFu) << 4, bo0 = (int)(b0 >> 8), be1 = (int)(b1 & 0xFFu) << 4, bo1 = (int)(b1 >> 8);
                v[0] = ae0 * cs[0][0] + ao0 * cs[1][0] + be0 * cs[2][0] + bo0 * cs[3][0];
                v[1] = ae0 * cs[0][1] + ao0 * cs[1][1] + be0 * cs[2][1] + bo0 * cs[3][1];
                v[2] = ae1 * cs[0][2] + ao1 * cs[1][2] + be1 * cs[2][2] + bo1 * cs[3][2];
                v[3] = ae1 * cs[0][3] + ao1 * cs[1][3] + be1 * cs[2][3] + bo1 * cs[3][3];
            }
            const bool up2 = (t & 2) != 0;   // row g + 8 ends in the lanes with t >= 2
            const uint32_t hx = up2 ? h1.x : h0.x;
            const float d16 = half_bits_to_float((uint16_t)(hx & 0xffffu)) * 0.0625f;
            const float dmin = half_bits_to_float((uint16_t)(hx >> 16));
            if (TP == 2) {
                // sum over the four slots (lanes t = 0..3); lane t ends with (row g + 8 (t>>1), token t & 1)
                const int ka = (up2 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, up2 ? v[0] : v[2], 2);
                const int kb = (up2 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, up2 ? v[1] : v[3], 2);
                const bool up1 = (t & 1) != 0;
                const int k = (up1 ? kb : ka) + __shfl_xor_sync(0xffffffffu, up1 ? ka : kb, 1);
                // columns 2t, 2t+1 of the mins product: high and low digit of token t & 1
                int cm[4];
                mma_u8s8_k32(cm, am0, am1, 0u, 0u, G.bm[0], 0u);
                const int imin = up2 ? 64 * cm[2] + cm[3] : 64 * cm[0] + cm[1];
                acc[mt][0] = G.dx[0] * (d16 * (float)k - dmin * (float)imin);
            } else {
                // sum over the two slots (lanes t, t ^ 2); the lane keeps (row g + 8 (t>>1), tokens 2 (t&1), 2 (t&1) + 1)
                const int k0 = (up2 ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, up2 ? v[0] : v[2], 2);
                const int k1 = (up2 ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, up2 ? v[1] : v[3], 2);
                int ch[4], cl[4];   // columns = tokens (n & 3): 2t, 2t+1 -> tokens 2 (t&1), 2 (t&1) + 1
                mma_u8s8_k32(ch, am0, am1, 0u, 0u, G.bm[0], 0u);
                mma_u8s8_k32(cl, am0, am1, 0u, 0u, G.bm[1], 0u);
                const int m0 = up2 ? 64 * ch[2] + cl[2] : 64 * ch[0] + cl[0];
                const int m1 = up2 ? 64 * ch[3] + cl[3] : 64 * ch[1] + cl[1];
                acc[mt][0] = G.dx[0] * (d16 * (float)k0 - dmin * (float)m0);
                acc[mt][1] = G.dx[1] * (d16 * (float)k1 - dmin * (float)m1);
            }
        }
    }
    // partial sums of this warp's block column into its own bytes of the first eight gate rows of the slot: value
    // idx of matrix mt = 16 TP mt + TP (row in the item) + token, at row idx >> 5, word idx & 31 of the warp's 144 bytes
    __syncwarp();
    {
        uint8_t *mine = stage + Q4_K_BYTES * warp;
        auto at = [&](int idx) -> uint8_t * { return mine + q4k_row_off(idx >> 5) + (idx & 31) * 4; };
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            if (TP == 2) {
                *reinterpret_cast<float *>(at(mt * 32 + (ra + 2 * (t >> 1)) * 2 + (t & 1))) = acc[mt][0];
            } else if (TP == 4) {
                *reinterpret_cast<float2 *>(at(mt * 64 + (ra + 2 * (t >> 1)) * 4 + 2 * (t & 1))) = make_float2(acc[mt][0], acc[mt][1]);
            } else {
                *reinterpret_cast<float2 *>(at(mt * 128 + ra * 8 + 2 * t)) = make_float2(acc[mt][0], acc[mt][1]);
                *reinterpret_cast<float2 *>(at(mt * 128 + rb * 8 + 2 * t)) = make_float2(acc[mt][2], acc[mt][3]);
            }
        }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
        constexpr int TPV = 8 / TP;   // threads per value, each adding TP of the eight partial sums
        const int mt = lane >> 4, part = lane % TPV;
        const int idx = mt * 16 * TP + warp * (16 / TPV) + (lane & 15) / TPV;
        const uint8_t *src = stage + q4k_row_off(idx >> 5) + (idx & 31) * 4 + Q4_K_BYTES * TP * part;
        // the eight partial sums are added as one balanced tree whatever TP is, so that a token's result does not
        // depend on how many tokens shared its group (the order of an expert's token list is not fixed between runs)
        float pv[TP];
#pragma unroll
        for (int w = 0; w < TP; w++) pv[w] = *reinterpret_cast<const float *>(src + Q4_K_BYTES * w);
#pragma unroll
        for (int st = 1; st < TP; st *= 2)
#pragma unroll
            for (int w = 0; w < TP; w += 2 * st) pv[w] += pv[w + st];
        float v = pv[0];
        if (TPV >= 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
        if (TPV >= 4) v += __shfl_xor_sync(0xffffffffu, v, 2);
        const float up = __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane < 16 && part == 0 && G.r_orow >= 0 && compute)
            A.out[(size_t)G.r_orow * A.rows_total + chunk * 16 + G.r_row] = v / (1.f + expf(-v)) * up;   // silu(gate) * up
    }
}

// The items of one (expert, token group) starting at `cur` (item `it` of the CTA).
template <int TP>
__device__ inline void gu_run_group(const GemvArgs &A, uint8_t *ring, const MmaWork &work, MmaCursor &cur, int &it, int n_items,
                                    bool is_sh, int my_row, int t0, int cnt, int warp, int lane, bool &failed, LookAhead &la,
                                    int &items_in_slot)
{
    GuGroup<TP> G;
    gu_load_group<TP>(A, is_sh, my_row, t0, cnt, warp, lane, G);
    const int slot = cur.slot, group = cur.group;
    while (it < n_items && cur.slot == slot && cur.group == group) {
        const int s = it % NSTAGE;
        const uint32_t use = (uint32_t)(it / NSTAGE);
        // a wait that runs out is recorded; the warp keeps walking its items (and meeting the barriers
        // it shares with the other warps) without computing
        if (!failed && A.debug != 2 && !mbar_wait(ring_full(ring, s), use & 1, A.max_polls)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 18, it);
            failed = true;
        }
        gu_item<TP>(A, ring_stage(ring, s, A.stage_bytes), G, cur.chunk, !failed && A.debug != 1, warp, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(ring_empty(ring, s));
        la.advance(A, work, lane);
        work.advance(cur);
        it++;
        items_in_slot++;
    }
}

// The compute warps' side: items [it, n_items) of this CTA starting at `cur`.
__device__ inline bool run_items_q4k_mma(const GemvArgs &A, uint8_t *ring, const MmaWork &work, MmaCursor cur, int n_items,
                                         int &it, int warp, int lane)
{
    LookAhead la;
    la.slot = la.group = -1;
    la.step = 3;
    bool failed = false;
    // PMOE_DEBUG=6 (test of the bounded waits): CTA 0 first waits on a barrier nothing ever arrives at; the wait runs
    // out, the status word gets PMOE_ERR_TIMEOUT and the warps walk their items without computing, as after any
    // expired wait
    if (A.debug == 6 && blockIdx.x == 0 && !mbar_wait(ring_full(ring, 2 * NSTAGE), 0, A.max_polls)) {
        set_status(A.status, PMOE_ERR_TIMEOUT, 19, 0);
        failed = true;
    }
    // progress bookkeeping for the fused re-quantisation: a routed expert is finished as a whole (all its groups),
    // the shared expert group by group (its eight rows are quantised by whoever completes the group)
    int cur_slot = -1, cur_group = -1, items_in_slot = 0, slot_groups = 0, slot_m = 0, slot_off = 0;
    bool slot_sh = false;
    auto leave = [&]() {
        if (cur_slot < 0 || (slot_sh ? A.quant_dt_s : A.quant_dt_r) == 0) return;
        if (slot_sh) {
            const int first = GEMV_TG_MMA * cur_group;
            finish_slot(A, A.e_local + 1 + cur_group, items_in_slot, work.cpe, true, nullptr,
                        slot_m - first < GEMV_TG_MMA ? slot_m - first : GEMV_TG_MMA, warp, lane, first);
        } else {
            finish_slot(A, cur_slot, items_in_slot, work.cpe * slot_groups, false, A.g.pairs + slot_off, slot_m, warp, lane);
        }
    };
    while (it < n_items) {
        const bool is_sh = cur.slot >= work.n_active;
        const int t0 = GEMV_TG_MMA * cur.group;
        int m, off = 0, my_row = -1;
        if (is_sh) {
            m = A.sh_count;
        } else if (la.ready(work, cur.slot, cur.group)) {
            m = la.m;
            off = la.off;
            my_row = la.row;
        } else {
            const int e = A.g.active[cur.slot];
            m = A.g.count[e];
            off = A.g.offset[e];
            const int i = t0 + (lane & 7);
            if (i < m) my_row = A.g.pairs[off + i];
        }
        if (cur.slot != cur_slot || is_sh) {
            leave();
            items_in_slot = 0;
            cur_slot = cur.slot;
            slot_groups = cur.groups;
            slot_sh = is_sh;
            slot_m = m;
            slot_off = off;
        }
        cur_group = cur.group;
        la.start(cur);
        const int cnt = m - t0 < GEMV_TG_MMA ? m - t0 : GEMV_TG_MMA;
        if (cnt <= 2) gu_run_group<2>(A, ring, work, cur, it, n_items, is_sh, my_row, t0, cnt, warp, lane, failed, la, items_in_slot);
        else if (cnt <= 4) gu_run_group<4>(A, ring, work, cur, it, n_items, is_sh, my_row, t0, cnt, warp, lane, failed, la, items_in_slot);
        else gu_run_group<8>(A, ring, work, cur, it, n_items, is_sh, my_row, t0, cnt, warp, lane, failed, la, items_in_slot);
    }
    leave();
    return !failed;
}

// ---------------------------------------------------------------- a Q8_0 shared expert beside the tensor-core items
// A Q8_0 shared expert over SHARED_MMA_MIN tokens or more is served by a tenth warp of every CTA, in the shadow
// of the routed experts' stream: the shared expert is small (it stays in L2), but a job -- 16 rows x 8 tokens over
// the whole K, one block per mma.m16n8k32 -- is a chain of L2 round trips, so it belongs beside the memory-bound
// work, not after it.  The jobs are numbered (16-row tile, 8-token tile), token tile fastest, and every CTA's warp
// takes an equal share; weights and activations are read straight from global memory.  For gate/up each token
// tile has a completion counter (behind the per-expert ones): the warp that finishes a tile's last job
// re-quantises those eight activated rows for the down projection.
constexpr int SHW_WARP = GEMV_WARPS + 1;
constexpr int SHW_THREADS = GEMV_THREADS + 32;

template <int NMAT> __device__ inline void q80_shared_warp(const GemvArgs &A, int lane)
{
    using C = Cfg<PMOE_Q8_0, NMAT>;
    constexpr int KB = C::K / QK8_0;
    const int g = lane >> 2, t = lane & 3;
    const int m = A.sh_count, ntiles = (m + 7) / 8;
    const int tiles16 = NMAT == 2 ? A.rows_total / 8 : A.rows_total / 16;   // gate/up: 8 gate + 8 up rows per tile
    const long total = (long)tiles16 * ntiles;
    const long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
    const QAct &in = A.in_s;
    const size_t row0 = NMAT == 2 ? (size_t)A.sh_begin : (size_t)A.n * A.top_k + A.sh_begin;  // activation row of token 0
    const size_t out0 = (size_t)A.n * A.top_k + A.sh_begin;                                   // output row of token 0
    const bool fuse_quant = NMAT == 2 && A.quant_dt_s != 0;
    if (A.debug == 1) return;
    for (long j = lo; j < hi; j++) {
        const int tile = (int)(j / ntiles), nt = (int)(j - (long)tile * ntiles);
        // fragment rows g and g + 8: gate row and up row 8*tile + g, or down rows 16*tile + g, + 8
        const uint8_t *r0 = A.sw0 + (size_t)(NMAT == 2 ? 8 * tile + g : 16 * tile + g) * C::ROW_BYTES;
        const uint8_t *r1 = NMAT == 2 ? A.sw1 + (size_t)(8 * tile + g) * C::ROW_BYTES : r0 + 8 * C::ROW_BYTES;
        // B column g = token 8 nt + g; C columns 2t, 2t+1 = tokens 8 nt + 2t (+1).  Columns past the last token
        // read token 0's rows; their sums are never stored.
        const int tok_b = nt * 8 + g, tok_c = nt * 8 + 2 * t;
        const bool c0_ok = tok_c < m, c1_ok = tok_c + 1 < m;
        const int8_t *xq = in.qs + (row0 + (tok_b < m ? tok_b : 0)) * C::K + 8 * t;
        const float *dx0 = in.d + (row0 + (c0_ok ? tok_c : 0)) * KB;
        const float *dx1 = in.d + (row0 + (c1_ok ? tok_c + 1 : 0)) * KB;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int kb = 0; kb < KB; kb += 8) {
            // every load of eight blocks is in flight before the first product: one round trip to L2 per step
            uint32_t a[8][4];
            uint2 bq[8];
            uint16_t dw[8][2];
            float4 x0[2], x1[2];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint8_t *p0 = r0 + (kb + i) * Q8_0_BYTES, *p1 = r1 + (kb + i) * Q8_0_BYTES;
                // the lane's share of K is bytes 8t..8t+7 of the block, for the weights and the activations alike;
                // kb is a multiple of 8: even blocks start on a word boundary (their quants do not), odd ones 2 bytes off
                if (i & 1) {
                    mma_load_row<true>(p0 + 2 + 8 * t, a[i][0], a[i][2]);
                    mma_load_row<true>(p1 + 2 + 8 * t, a[i][1], a[i][3]);
                } else {
                    mma_load_row<false>(p0 + 2 + 8 * t, a[i][0], a[i][2]);
                    mma_load_row<false>(p1 + 2 + 8 * t, a[i][1], a[i][3]);
                }
                dw[i][0] = *reinterpret_cast<const uint16_t *>(p0);
                dw[i][1] = *reinterpret_cast<const uint16_t *>(p1);
                bq[i] = *reinterpret_cast<const uint2 *>(xq + (kb + i) * QK8_0);
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                x0[h] = *reinterpret_cast<const float4 *>(dx0 + kb + 4 * h);
                x1[h] = *reinterpret_cast<const float4 *>(dx1 + kb + 4 * h);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t b[2] = {bq[i].x, bq[i].y};
                int c[4];
                mma_s8_16x8x32(c, a[i], b);
                const float dw0 = half_bits_to_float(dw[i][0]), dw1 = half_bits_to_float(dw[i][1]);
                const float4 &xa = x0[i >> 2], &xb = x1[i >> 2];
                const float xs0 = (i & 3) == 0 ? xa.x : (i & 3) == 1 ? xa.y : (i & 3) == 2 ? xa.z : xa.w;
                const float xs1 = (i & 3) == 0 ? xb.x : (i & 3) == 1 ? xb.y : (i & 3) == 2 ? xb.z : xb.w;
                acc[0] += (dw0 * xs0) * (float)c[0];
                acc[1] += (dw0 * xs1) * (float)c[1];
                acc[2] += (dw1 * xs0) * (float)c[2];
                acc[3] += (dw1 * xs1) * (float)c[3];
            }
        }
        if (NMAT == 2) {
            const int row = 8 * tile + g;
            const float v0 = acc[0] / (1.f + expf(-acc[0])) * acc[2];  // silu(gate) * up
            const float v1 = acc[1] / (1.f + expf(-acc[1])) * acc[3];
            if (c0_ok) A.out[(out0 + tok_c) * A.rows_total + row] = v0;
            if (c1_ok) A.out[(out0 + tok_c + 1) * A.rows_total + row] = v1;
        } else {
            const int row = 16 * tile + g;
            if (c0_ok) {
                const float sc = A.scale_s[A.sh_begin + tok_c];
                float *o = A.out + (out0 + tok_c) * A.rows_total + row;
                o[0] = acc[0] * sc;
                o[8] = acc[2] * sc;
            }
            if (c1_ok) {
                const float sc = A.scale_s[A.sh_begin + tok_c + 1];
                float *o = A.out + (out0 + tok_c + 1) * A.rows_total + row;
                o[0] = acc[1] * sc;
                o[8] = acc[3] * sc;
            }
        }
        if (fuse_quant) {
            __threadfence();   // every lane's rows before the counter update, the reader's fence after it
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                const int old = atomicAdd(&A.slot_done[A.e_local + 1 + nt], 1);
                last = old + 1 == tiles16;
                if (last) A.slot_done[A.e_local + 1 + nt] = 0;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last && A.debug != 3) {
                __threadfence();
                const bool kq = is_kquant(A.quant_dt_s);
                const int rows = m - 8 * nt < 8 ? m - 8 * nt : 8;
                for (int i = 0; i < rows; i++) {
                    const size_t r = out0 + 8 * nt + i;
                    warp_quant_row512(A.out + r * 512, kq, A.q8k_out, A.q80_out, r, lane);
                }
            }
        }
    }
}

// DT_S: type of the shared expert's gate/up matrices served by this launch (0 = none).  A Q4_K shared
// expert is one more slot of the tensor-core items; other types follow as items of the streaming kind.
template <int DT_S>
__global__ void __launch_bounds__(DT_S == PMOE_Q8_0 ? SHW_THREADS : GEMV_THREADS, 2) k_gate_up_q4k_mma(const GemvArgs A)
{
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ int s_prefix1[2];
    __shared__ MmaCursor s_first;
    __shared__ int s_items;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_dependents();

    MmaWork work;
    work.n_active = 0;
    work.cpe = A.rows_total / 16;
    work.groups_sh = (DT_S == PMOE_Q4_K && A.has_shared) ? (A.sh_count + GEMV_TG_MMA - 1) / GEMV_TG_MMA : 0;
    work.prefix = A.g.cost_prefix_mma;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(ring_full(ring, s), 1);
            mbar_init(ring_empty(ring, s), GEMV_WARPS);
        }
        mbar_init(ring_full(ring, 2 * NSTAGE), 1);   // never arrived at: the timeout test waits on it
        fence_mbar_init();
        s_prefix1[0] = s_prefix1[1] = 0;
    }
    mma_plan(work, A, &s_first, &s_items);
    __syncthreads();
    const int n_mma = s_items;
    const MmaCursor first = s_first;

    // items of the streaming kind for a shared expert of another type: an equal share of their cost
    constexpr bool STREAM_SH = DT_S != 0 && DT_S != PMOE_Q4_K;
    constexpr int DT_S1 = STREAM_SH ? DT_S : PMOE_Q8_0;
    using CS = Cfg<DT_S1, 2>;
    Plan plan;
    Cursor scur{0, 0};
    int n_sh = 0;
    // a Q8_0 shared expert has a warp of its own (PMOE_SHW_MIN: from that many tokens on; below, streaming items follow)
    const bool shared_warp = DT_S == PMOE_Q8_0 && A.has_shared && A.sh_count >= A.shw_min;
    if (STREAM_SH && A.has_shared) {
        plan.n_active = 0;
        plan.has_shared = 1;
        plan.cpe_r = plan.cpe_s = A.rows_total / CS::ROWS;
        plan.shared_mma = false;
        plan.cost_shared = (A.sh_count + CS::TGK - 1) / CS::TGK;
        plan.prefix = s_prefix1;
        if (!shared_warp) {
            const long total = plan.total_cost();
            scur = plan.find(total * blockIdx.x / gridDim.x);
            const Cursor last = plan.find(total * (blockIdx.x + 1) / gridDim.x);
            n_sh = plan.index(last) - plan.index(scur);
        }
    }
    if (DT_S == PMOE_Q8_0 && warp == SHW_WARP) {   // the shared expert's warp
        if (shared_warp) q80_shared_warp<2>(A, lane);
        return;
    }
    if (n_mma + n_sh <= 0) return;

    if (warp == GEMV_WARPS) {   // the producer warp: eight lanes copy four rows of an item each
        if (A.debug == 2) return;
        MmaCursor pc = first;
        int issued = 0;
        bool ok = true;
        for (; issued < n_mma; issued++) {
            const int s = issued % NSTAGE;
            const uint32_t use = (uint32_t)(issued / NSTAGE);
            if (use > 0) {
                // the slot must have been released, and its previous copy must have landed: warps that gave up
                // waiting release slots early, and a barrier must not be armed twice in one phase
                int w = 1;
                if (lane == 0)
                    w = mbar_wait(ring_empty(ring, s), (use - 1) & 1, A.max_polls) &&
                                mbar_wait(ring_full(ring, s), (use - 1) & 1, A.max_polls)
                            ? 1 : 0;
                w = __shfl_sync(0xffffffffu, w, 0);
                if (!w) {
                    if (lane == 0) set_status(A.status, PMOE_ERR_TIMEOUT, 23, issued);
                    ok = false;
                    break;
                }
            }
            // lanes 0..7 copy four consecutive rows each: lane = 4 * matrix + quad
            const uint8_t *base;
            if (pc.slot < work.n_active) base = (lane < 4 ? A.w0 : A.w1) + (size_t)A.g.active[pc.slot] * A.expert_bytes;
            else base = lane < 4 ? A.sw0 : A.sw1;
            uint64_t *full = ring_full(ring, s);
            if (lane == 0) mbar_expect_tx(full, 32 * Q4K_ROW);
            __syncwarp();
            if (lane < 8)
                bulk_g2s(ring_stage(ring, s, A.stage_bytes) + (lane >> 2) * Q4K_TILE + (lane & 3) * Q4K_QUAD,
                         base + (size_t)(pc.chunk * 16 + 4 * (lane & 3)) * Q4K_ROW, 4 * Q4K_ROW, full);
            work.advance(pc);
        }
        if (lane == 0) {
            if (STREAM_SH && ok && n_sh > 0) {
                Producer<DT_S1, DT_S1, 2> prod{A, plan, ring, scur, issued, n_mma + n_sh};
                for (int i = 0; i < n_sh; i++)
                    if (!prod.issue_next()) { prod.issued--; break; }
                issued = prod.issued;
            }
            drain_ring(ring, issued, A.max_polls);
        }
        return;
    }
    int it = 0;
    bool ok = run_items_q4k_mma(A, ring, work, first, n_mma, it, warp, lane);
    if constexpr (STREAM_SH) {
        if (ok && n_sh > 0) run_items<DT_S1, 2>(A, ring, plan, true, scur, 1, it, n_mma + n_sh, A.in_s, warp, lane);
    }
}

template <int DT_S> static cudaError_t launch_q4k_mma_t(const GemvArgs &A, cudaStream_t s)
{
    constexpr size_t smem = 128 + (size_t)NSTAGE * MMA_STAGE_BYTES;
    auto kern = k_gate_up_q4k_mma<DT_S>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaError_t e = launch_pdl(kern, dim3(2 * sm_count()), dim3(DT_S == PMOE_Q8_0 ? SHW_THREADS : GEMV_THREADS), smem, s, A);
    count_launch();
    return e;
}


// ---------------------------------------------------------------- Q6_K down on the tensor cores
// The down projection for Q6_K experts (rows of K = 512 = two blocks of 210 bytes) with the dot products
// on the tensor cores.  A 16-weight sub-block -- the span of one int8 scale -- never shares an
// accumulator column with another one, so the integer sub-block sums stay exact and meet their scales
// as integers, like the dp4a path:
//
//   up to 2 tokens   m16n8k32, the eight accumulator columns are (sub-block slot 0..3) x (token 0..1):
//                    an instruction covers two sub-blocks (low / high nibble streams of the same ql
//                    bytes) and a token's activations are non-zero only in the K half and columns of
//                    its own slot, so two instructions fill one accumulator with four sub-block sums;
//   up to 4 tokens   m16n8k32, columns are (slot 0..1) x (token 0..3), one accumulator per instruction;
//   up to 8 tokens   m16n8k16, one sub-block per instruction, columns are the tokens.
//
// Quants are used as the unsigned 6-bit values; the offset -32 comes back as -32 * sum_j sc_j * bsum_j
// from the Q8_K partial sums (one sub-block = one partial sum), through one or two more instructions
// whose A operand is the row's sixteen scales and whose B operand holds the partial sums split into
// two signed byte digits (bsum = 64 h + l).
//
// An item is 64 rows of one expert (26 880 contiguous bytes, one bulk copy).  The eight compute warps
// form two teams of four; a team takes every other item and each of its warps one 16-row tile over
// the whole K, so no partial sums cross warps and the warps of a CTA never meet at a barrier.  Rows
// are 420 bytes apart in shared memory: the eight rows of a fragment fall into different banks.  The
// second block of a row starts 2 bytes off a word; its words are read as two halves.
constexpr int Q6K_ROW = 2 * Q6_K_BYTES;        // 420
constexpr int DM_ROWS = 64;
constexpr int DM_ITEM = DM_ROWS * Q6K_ROW;     // 26 880
constexpr int DM_NSTAGE = 4;
constexpr int DM_HDR = 256;                    // barriers of both phases live in front of the stages
constexpr int DM_RING2 = 64;                   // base of the streaming-kind ring (shared expert of another type)
constexpr size_t DM_SMEM = DM_HDR + (size_t)DM_NSTAGE * DM_ITEM > DM_RING2 + 128 + (size_t)NSTAGE * STAGE_BYTES
                               ? DM_HDR + (size_t)DM_NSTAGE * DM_ITEM
                               : DM_RING2 + 128 + (size_t)NSTAGE * STAGE_BYTES;
static_assert(DM_ITEM % 16 == 0 && DM_HDR % 128 == 0, "bulk copies need 16-byte alignment");

__device__ inline uint64_t *dm_full(uint8_t *smem, int s) { return reinterpret_cast<uint64_t *>(smem) + s; }
__device__ inline uint64_t *dm_empty(uint8_t *smem, int s) { return reinterpret_cast<uint64_t *>(smem) + DM_NSTAGE + s; }
__device__ inline uint8_t *dm_stage(uint8_t *smem, int s) { return smem + DM_HDR + s * DM_ITEM; }

__device__ inline void mma_s8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                    uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ inline void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ inline void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// a word of block B of a row: block 0 starts on a word boundary, block 1 two bytes off one
template <int B> __device__ inline uint32_t q6_word(const uint8_t *p)
{
    if (B == 0) return *reinterpret_cast<const uint32_t *>(p);
    return lds_u32_a2(p);
}

// byte i of w, sign-extended: one permute whose upper three selectors replicate the byte's sign
// (i is a constant once the caller's loops are unrolled)
__device__ inline int sbyte(uint32_t w, int i)
{
    int d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"(0x8880u + 0x1111u * (uint32_t)i));
    return d;
}

// Four packed int16 partial sums -> their high (v >> 6) or low (v & 63) digits as four bytes.
__device__ inline uint32_t bsum_digits(uint2 v, bool low)
{
    const int s[4] = {(int)(int16_t)(v.x & 0xffffu), (int)(int16_t)(v.x >> 16), (int)(int16_t)(v.y & 0xffffu),
                      (int)(int16_t)(v.y >> 16)};
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) o |= (uint32_t)((low ? (s[i] & 63) : (s[i] >> 6)) & 0xFF) << (8 * i);
    return o;
}

// The unsigned 6-bit quants of the two sub-blocks that share the ql word `ql`: stream SA (low nibbles, high
// bits at 2*SA of qh) and stream SA + 2 (high nibbles, high bits at 4 + 2*SA).
template <int SA> __device__ inline void q6_unpack(uint32_t ql, uint32_t qh, uint32_t &lo, uint32_t &hi)
{
    lo = (ql & 0x0F0F0F0Fu) | ((qh << (4 - 2 * SA)) & 0x30303030u);
    hi = ((ql >> 4) & 0x0F0F0F0Fu) | ((SA == 0 ? qh : qh >> 2) & 0x30303030u);
}

// What a group of up to TP tokens of one expert leaves in a lane's registers.
template <int TP> struct DmGroup {
    static constexpr int NX = TP == 2 ? 8 : TP == 4 ? 16 : 32;   // activation words
    static constexpr int NF = TP == 2 ? 1 : TP == 4 ? 2 : 4;     // results a lane ends with
    static constexpr int NT = TP == 8 ? 2 : NF;                  // tokens those results belong to
    uint32_t x[NX];
    uint32_t bs[TP == 2 ? 1 : TP == 4 ? 2 : 4];   // partial-sum digits
    float dx[NT][2];                              // activation scale per final token and block
    int orow[NT];                                 // output row per final token (-1: none)
    float scale[NT];
};

// my_row: pair id of token (lane & 7) of the group (routed experts).  Every lane of the warp calls this; the
// shuffles that hand a token's row to the lanes that need it run before anything diverges.
template <int TP>
__device__ inline void dm_load_group(const GemvArgs &A, bool is_sh, int my_row, int t0, int cnt, int lane, DmGroup<TP> &G)
{
    const int g = lane >> 2, t = lane & 3;
    const QAct &in = is_sh ? A.in_s : A.in_r;
    // row of the quantised activation (and of the output) of token i of the group
    auto row_of = [&](int i) -> size_t {
        const int p = __shfl_sync(0xffffffffu, my_row, i & 7);
        return is_sh ? (size_t)A.n * A.top_k + A.sh_begin + t0 + i : (size_t)p;
    };
    const int tok_b = TP == 2 ? (g & 1) : TP == 4 ? (g & 3) : g;            // token of the lane's B column
    const int tok_s = TP == 2 ? ((g >> 1) & 1) : TP == 4 ? (g & 3) : g;     // token of its partial-sum column
    const size_t row_b = row_of(tok_b), row_s = row_of(tok_s);
    size_t row_f[DmGroup<TP>::NT];
#pragma unroll
    for (int j = 0; j < DmGroup<TP>::NT; j++) row_f[j] = row_of(TP == 2 ? (t & 1) : TP == 4 ? 2 * (t & 1) + j : 2 * t + j);

    // ---- B operands of the main products
#pragma unroll
    for (int i = 0; i < DmGroup<TP>::NX; i++) G.x[i] = 0;
    if (tok_b < cnt) {
        const int8_t *xp = in.qs + row_b * 512 + 4 * t;
        if (TP == 2) {          // x[4b + a]: sub-blocks 8*m_own + 4*ab_own + a, a = 0..3
            const int s0 = 8 * (g >> 2) + 4 * ((g >> 1) & 1);
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int a = 0; a < 4; a++) G.x[4 * b + a] = *reinterpret_cast<const uint32_t *>(xp + 256 * b + 16 * (s0 + a));
        } else if (TP == 4) {   // x[8b + 2a + m]: sub-block 8*m + 4*ab_own + a
            const int s0 = 4 * (g >> 2);
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int a = 0; a < 4; a++)
#pragma unroll
                    for (int m = 0; m < 2; m++)
                        G.x[8 * b + 2 * a + m] = *reinterpret_cast<const uint32_t *>(xp + 256 * b + 16 * (8 * m + s0 + a));
        } else {                // x[16b + S]
#pragma unroll
            for (int b = 0; b < 2; b++)
#pragma unroll
                for (int S = 0; S < 16; S++) G.x[16 * b + S] = *reinterpret_cast<const uint32_t *>(xp + 256 * b + 16 * S);
        }
    }
    // ---- B operands of the offset products: digits of the partial sums 4t .. 4t+3 of one block of one token
    if (TP == 2) {          // column g = (block g>>2, token (g>>1)&1, digit g&1)
        G.bs[0] = 0;
        if (tok_s < cnt)
            G.bs[0] = bsum_digits(*reinterpret_cast<const uint2 *>(in.bsums + row_s * 32 + 16 * (g >> 2) + 4 * t), g & 1);
    } else if (TP == 4) {   // column g = (block g>>2, token g&3); bs[0] high digits, bs[1] low digits
        G.bs[0] = G.bs[1] = 0;
        if (tok_s < cnt) {
            const uint2 v = *reinterpret_cast<const uint2 *>(in.bsums + row_s * 32 + 16 * (g >> 2) + 4 * t);
            G.bs[0] = bsum_digits(v, false);
            G.bs[1] = bsum_digits(v, true);
        }
    } else {                // column g = token g; bs[2b] high, bs[2b+1] low digits of block b
#pragma unroll
        for (int i = 0; i < 4; i++) G.bs[i] = 0;
        if (tok_s < cnt) {
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const uint2 v = *reinterpret_cast<const uint2 *>(in.bsums + row_s * 32 + 16 * b + 4 * t);
                G.bs[2 * b] = bsum_digits(v, false);
                G.bs[2 * b + 1] = bsum_digits(v, true);
            }
        }
    }
    // ---- what the lane's final values need: their tokens' scales and output rows
#pragma unroll
    for (int j = 0; j < DmGroup<TP>::NT; j++) {
        const int tok = TP == 2 ? (t & 1) : TP == 4 ? 2 * (t & 1) + j : 2 * t + j;
        G.orow[j] = -1;
        G.scale[j] = 0.f;
        G.dx[j][0] = G.dx[j][1] = 0.f;
        if (tok < cnt) {
            const size_t r = row_f[j];
            G.orow[j] = (int)r;
            G.dx[j][0] = in.d[r * 2];
            G.dx[j][1] = in.d[r * 2 + 1];
            G.scale[j] = is_sh ? A.scale_s[A.sh_begin + t0 + tok] : A.scale_r[r];
        }
    }
}

// Block b (compile-time: the second block of a row is read with half-word loads) of one tile: its sixteen
// sub-block products, scales and offset, added to the lane's results.
template <int TP, int b>
__device__ inline void dm_block(const uint8_t *r0, const uint8_t *r1, const DmGroup<TP> &G, const uint32_t (&scw)[2][2],
                                const int (&corr)[2][4], int lane, float (&f)[DmGroup<TP>::NF])
{
    const int g = lane >> 2, t = lane & 3;
    const uint8_t *p0 = r0 + b * Q6_K_BYTES, *p1 = r1 + b * Q6_K_BYTES;
    int iacc[4] = {0, 0, 0, 0};   // (row g, token pair), (row g + 8, token pair)
    if (TP == 2) {
        // lane's accumulator columns 2t, 2t+1 = slot t, tokens 0, 1; slot t of accumulator a = sub-block 4t + a
        const uint32_t own0 = (g >> 2) == 0 ? 0xffffffffu : 0u, own1 = ~own0;   // instruction m: the lane's data or zeros
        const bool lowhalf = ((g >> 1) & 1) == 0;                               // its slot sits in the K half 0..15
#pragma unroll
        for (int a = 0; a < 4; a++) {
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const int qoff = 64 * m + 32 * (a >> 1) + 16 * (a & 1) + 4 * t, hoff = 128 + 32 * m + 16 * (a & 1) + 4 * t;
                uint32_t a0, a1, a2, a3;
                if ((a >> 1) == 0) {
                    q6_unpack<0>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), a0, a2);
                    q6_unpack<0>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), a1, a3);
                } else {
                    q6_unpack<1>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), a0, a2);
                    q6_unpack<1>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), a1, a3);
                }
                const uint32_t xv = G.x[4 * b + a] & (m == 0 ? own0 : own1);
                mma_u8s8_k32_acc(c, a0, a1, a2, a3, lowhalf ? xv : 0u, lowhalf ? 0u : xv);
            }
            const int s0 = sbyte(scw[b][0], a);
            const int s1 = sbyte(scw[b][1], a);
            iacc[0] += c[0] * s0; iacc[1] += c[1] * s0; iacc[2] += c[2] * s1; iacc[3] += c[3] * s1;
        }
        // the offset of (block t>>1, token t&1) sits in this lane: into the matching partial sums
        if ((t >> 1) == b) {
            const int o0 = -32 * corr[0][0], o1 = -32 * corr[0][1];
            iacc[0] += (t & 1) ? 0 : o0; iacc[1] += (t & 1) ? o0 : 0;
            iacc[2] += (t & 1) ? 0 : o1; iacc[3] += (t & 1) ? o1 : 0;
        }
        // sum over the four slots (lanes t = 0..3); lane t ends with value t = (row t>>1, token t&1)
        const bool up2 = (t & 2) != 0;
        int ka = (up2 ? iacc[2] : iacc[0]) + __shfl_xor_sync(0xffffffffu, up2 ? iacc[0] : iacc[2], 2);
        int kb = (up2 ? iacc[3] : iacc[1]) + __shfl_xor_sync(0xffffffffu, up2 ? iacc[1] : iacc[3], 2);
        const bool up1 = (t & 1) != 0;
        const int k = (up1 ? kb : ka) + __shfl_xor_sync(0xffffffffu, up1 ? ka : kb, 1);
        const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>((up2 ? p1 : p0) + 208));
        f[0] += (dw * G.dx[0][b]) * (float)k;
    } else if (TP == 4) {
        // one accumulator per instruction; lane's columns = slot t>>1, tokens 2(t&1), 2(t&1)+1;
        // slot (t>>1) of instruction (a, m) = sub-block 8m + 4(t>>1) + a
        const bool lowhalf = (g >> 2) == 0;
        uint32_t scm[2][2];   // [m][row]: scale bytes 8m + 4(t>>1) .. +3
#pragma unroll
        for (int m = 0; m < 2; m++) {
            scm[m][0] = q6_word<b>(p0 + 192 + 8 * m + 4 * (t >> 1));
            scm[m][1] = q6_word<b>(p1 + 192 + 8 * m + 4 * (t >> 1));
        }
#pragma unroll
        for (int a = 0; a < 4; a++) {
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const int qoff = 64 * m + 32 * (a >> 1) + 16 * (a & 1) + 4 * t, hoff = 128 + 32 * m + 16 * (a & 1) + 4 * t;
                uint32_t a0, a1, a2, a3;
                if ((a >> 1) == 0) {
                    q6_unpack<0>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), a0, a2);
                    q6_unpack<0>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), a1, a3);
                } else {
                    q6_unpack<1>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), a0, a2);
                    q6_unpack<1>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), a1, a3);
                }
                int c[4] = {0, 0, 0, 0};
                const uint32_t xv = G.x[8 * b + 2 * a + m];
                mma_u8s8_k32_acc(c, a0, a1, a2, a3, lowhalf ? xv : 0u, lowhalf ? 0u : xv);
                const int s0 = sbyte(scm[m][0], a);
                const int s1 = sbyte(scm[m][1], a);
                iacc[0] += c[0] * s0; iacc[1] += c[1] * s0; iacc[2] += c[2] * s1; iacc[3] += c[3] * s1;
            }
        }
        if ((t >> 1) == b) {
#pragma unroll
            for (int i = 0; i < 4; i++) iacc[i] -= 32 * corr[0][i];
        }
        // sum over the two slots (lanes t, t ^ 2); lanes t < 2 keep row g, the others row g + 8
        const bool up2 = (t & 2) != 0;
        const int k0 = (up2 ? iacc[2] : iacc[0]) + __shfl_xor_sync(0xffffffffu, up2 ? iacc[0] : iacc[2], 2);
        const int k1 = (up2 ? iacc[3] : iacc[1]) + __shfl_xor_sync(0xffffffffu, up2 ? iacc[1] : iacc[3], 2);
        const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>((up2 ? p1 : p0) + 208));
        f[0] += (dw * G.dx[0][b]) * (float)k0;
        f[1] += (dw * G.dx[1][b]) * (float)k1;
    } else {
        // one sub-block per instruction; columns are the tokens
        uint32_t sca[4][2];   // all sixteen scales of both rows
#pragma unroll
        for (int w = 0; w < 4; w++) {
            sca[w][0] = q6_word<b>(p0 + 192 + 4 * w);
            sca[w][1] = q6_word<b>(p1 + 192 + 4 * w);
        }
#pragma unroll
        for (int m = 0; m < 2; m++) {
#pragma unroll
            for (int a = 0; a < 4; a++) {
                const int qoff = 64 * m + 32 * (a >> 1) + 16 * (a & 1) + 4 * t, hoff = 128 + 32 * m + 16 * (a & 1) + 4 * t;
                uint32_t lo0, hi0, lo1, hi1;
                if ((a >> 1) == 0) {
                    q6_unpack<0>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), lo0, hi0);
                    q6_unpack<0>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), lo1, hi1);
                } else {
                    q6_unpack<1>(q6_word<b>(p0 + qoff), q6_word<b>(p0 + hoff), lo0, hi0);
                    q6_unpack<1>(q6_word<b>(p1 + qoff), q6_word<b>(p1 + hoff), lo1, hi1);
                }
                // sub-blocks SA = 8m + a (low nibbles) and SB = 8m + 4 + a (high nibbles): scale words 2m and 2m + 1, byte a
                int c[4];
                mma_u8s8_k16(c, lo0, lo1, G.x[16 * b + 8 * m + a]);
                {
                    const uint32_t w0 = sca[2 * m][0], w1 = sca[2 * m][1];
                    const int s0 = sbyte(w0, a);
                    const int s1 = sbyte(w1, a);
                    iacc[0] += c[0] * s0; iacc[1] += c[1] * s0; iacc[2] += c[2] * s1; iacc[3] += c[3] * s1;
                }
                mma_u8s8_k16(c, hi0, hi1, G.x[16 * b + 8 * m + 4 + a]);
                {
                    const uint32_t w0 = sca[2 * m + 1][0], w1 = sca[2 * m + 1][1];
                    const int s0 = sbyte(w0, a);
                    const int s1 = sbyte(w1, a);
                    iacc[0] += c[0] * s0; iacc[1] += c[1] * s0; iacc[2] += c[2] * s1; iacc[3] += c[3] * s1;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) iacc[i] -= 32 * corr[b][i];
        const float dw0 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(p0 + 208));
        const float dw1 = half_bits_to_float(*reinterpret_cast<const uint16_t *>(p1 + 208));
        f[0] += (dw0 * G.dx[0][b]) * (float)iacc[0];
        f[1] += (dw0 * G.dx[1][b]) * (float)iacc[1];
        f[2] += (dw1 * G.dx[0][b]) * (float)iacc[2];
        f[3] += (dw1 * G.dx[1][b]) * (float)iacc[3];
    }
}

// One 16-row tile (rows r0 = tile row g, r1 = tile row g + 8 of the item in shared memory) against the group.
// out_col = index of tile row 0 in the output row.
template <int TP>
__device__ inline void dm_tile(const GemvArgs &A, const uint8_t *r0, const uint8_t *r1, const DmGroup<TP> &G, int out_col,
                               int lane)
{
    const int g = lane >> 2, t = lane & 3;
    float f[DmGroup<TP>::NF];
#pragma unroll
    for (int i = 0; i < DmGroup<TP>::NF; i++) f[i] = 0.f;

    // the rows' scale words and the offset products (both blocks)
    uint32_t scw[2][2];   // [block][row]: bytes 4t .. 4t+3 of the sixteen scales
    scw[0][0] = q6_word<0>(r0 + 192 + 4 * t);
    scw[0][1] = q6_word<0>(r1 + 192 + 4 * t);
    scw[1][0] = q6_word<1>(r0 + Q6_K_BYTES + 192 + 4 * t);
    scw[1][1] = q6_word<1>(r1 + Q6_K_BYTES + 192 + 4 * t);
    int corr[2][4];       // [block][(row, token) as in the accumulators]; TP 2 and 4: only the lane's block (t >> 1) is set
    if (TP == 2) {
        // column pair t = (high, low) digit of (block t>>1, token t&1)
        const int blk = g >> 2;
        int cm[4];
        mma_s8s8_k32(cm, scw[0][0], scw[0][1], scw[1][0], scw[1][1], blk == 0 ? G.bs[0] : 0u, blk == 1 ? G.bs[0] : 0u);
        corr[0][0] = 64 * cm[0] + cm[1];   // row g
        corr[0][1] = 64 * cm[2] + cm[3];   // row g + 8
    } else if (TP == 4) {
        // columns 2t, 2t+1 = (block t>>1, tokens 2(t&1), 2(t&1)+1)
        const int blk = g >> 2;
        int ch[4], cl[4];
        mma_s8s8_k32(ch, scw[0][0], scw[0][1], scw[1][0], scw[1][1], blk == 0 ? G.bs[0] : 0u, blk == 1 ? G.bs[0] : 0u);
        mma_s8s8_k32(cl, scw[0][0], scw[0][1], scw[1][0], scw[1][1], blk == 0 ? G.bs[1] : 0u, blk == 1 ? G.bs[1] : 0u);
#pragma unroll
        for (int i = 0; i < 4; i++) corr[0][i] = 64 * ch[i] + cl[i];
    } else {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            int ch[4], cl[4];
            mma_s8s8_k16(ch, scw[b][0], scw[b][1], G.bs[2 * b]);
            mma_s8s8_k16(cl, scw[b][0], scw[b][1], G.bs[2 * b + 1]);
#pragma unroll
            for (int i = 0; i < 4; i++) corr[b][i] = 64 * ch[i] + cl[i];
        }
    }

    dm_block<TP, 0>(r0, r1, G, scw, corr, lane, f);
    dm_block<TP, 1>(r0, r1, G, scw, corr, lane, f);

    // store: x routing weight (shared expert: x its sigmoid gate)
    if (TP == 2) {
        if (G.orow[0] >= 0) A.out[(size_t)G.orow[0] * A.rows_total + out_col + g + 8 * (t >> 1)] = f[0] * G.scale[0];
    } else if (TP == 4) {
#pragma unroll
        for (int j = 0; j < 2; j++)
            if (G.orow[j] >= 0) A.out[(size_t)G.orow[j] * A.rows_total + out_col + g + 8 * (t >> 1)] = f[j] * G.scale[j];
    } else {
#pragma unroll
        for (int j = 0; j < 2; j++)
            if (G.orow[j] >= 0) {
                A.out[(size_t)G.orow[j] * A.rows_total + out_col + g] = f[j] * G.scale[j];
                A.out[(size_t)G.orow[j] * A.rows_total + out_col + g + 8] = f[2 + j] * G.scale[j];
            }
    }
}

// The items of one (expert, token group) this team takes, starting at `cur` (item `it` of the CTA).
template <int TP>
__device__ inline void dm_run_group(const GemvArgs &A, uint8_t *smem, const MmaWork &work, MmaCursor &cur, int &it,
                                    int n_items, bool is_sh, int my_row, int t0, int cnt, int mtile, int lane,
                                    bool &failed, LookAhead &la)
{
    DmGroup<TP> G;
    dm_load_group<TP>(A, is_sh, my_row, t0, cnt, lane, G);
    const int g = lane >> 2;
    const int slot = cur.slot, group = cur.group;
    while (it < n_items && cur.slot == slot && cur.group == group) {
        const int s = it % DM_NSTAGE;
        const uint32_t use = (uint32_t)(it / DM_NSTAGE);
        // a wait that runs out is recorded; the warp keeps walking its items without computing, so that
        // the producer still sees its stages released
        if (!failed && A.debug != 2 && !mbar_wait(dm_full(smem, s), use & 1, A.max_polls)) {
            set_status(A.status, PMOE_ERR_TIMEOUT, 31, it);
            failed = true;
        }
        if (!failed && A.debug != 1) {
            const uint8_t *r0 = dm_stage(smem, s) + (16 * mtile + g) * Q6K_ROW;
            dm_tile<TP>(A, r0, r0 + 8 * Q6K_ROW, G, cur.chunk * DM_ROWS + 16 * mtile, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(dm_empty(smem, s));
        la.advance(A, work, lane);
        work.advance(cur);
        work.advance(cur);
        it += 2;
    }
}

// DT_S: type of the shared expert's down matrix served by this launch (0 = none).  A Q6_K shared expert is
// one more slot of the tensor-core items; other types follow as items of the streaming kind.
template <int DT_S>
__global__ void __launch_bounds__(DT_S == PMOE_Q8_0 ? SHW_THREADS : GEMV_THREADS, 2) k_down_q6k_mma(const GemvArgs A)
{
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_prefix1[2];
    __shared__ MmaCursor s_first;
    __shared__ int s_items;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The predecessor (gate/up or the re-quantisation) let this kernel start after its own wait: the expert
    // lists are complete, so the plan is made and the producer streams weights while the predecessor still
    // runs; only the compute warps wait, for the quantised activations.
    pdl_launch_dependents();

    uint8_t *ring2 = smem + DM_RING2;
    MmaWork work;
    work.n_active = 0;
    work.cpe = A.rows_total / DM_ROWS;
    work.groups_sh = (DT_S == PMOE_Q6_K && A.has_shared) ? (A.sh_count + GEMV_TG_MMA - 1) / GEMV_TG_MMA : 0;
    work.prefix = A.g.cost_prefix_mma;
    if (threadIdx.x == 0) {
        for (int s = 0; s < DM_NSTAGE; s++) {
            mbar_init(dm_full(smem, s), 1);
            mbar_init(dm_empty(smem, s), GEMV_WARPS / 2);
        }
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(ring_full(ring2, s), 1);
            mbar_init(ring_empty(ring2, s), GEMV_WARPS);
        }
        fence_mbar_init();
        s_prefix1[0] = s_prefix1[1] = 0;
    }
    mma_plan(work, A, &s_first, &s_items);
    __syncthreads();
    const int n_mma = s_items;
    const MmaCursor first = s_first;

    // items of the streaming kind for a shared expert of another type: an equal share of their cost
    constexpr bool STREAM_SH = DT_S != 0 && DT_S != PMOE_Q6_K;
    constexpr int DT_S1 = STREAM_SH ? DT_S : PMOE_Q8_0;
    using CS = Cfg<DT_S1, 1>;
    Plan plan;
    Cursor scur{0, 0};
    int n_sh = 0;
    // a Q8_0 shared expert has a warp of its own (PMOE_SHW_MIN: from that many tokens on; below, streaming items follow)
    const bool shared_warp = DT_S == PMOE_Q8_0 && A.has_shared && A.sh_count >= A.shw_min;
    if (STREAM_SH && A.has_shared && !shared_warp) {
        plan.n_active = 0;
        plan.has_shared = 1;
        plan.cpe_r = plan.cpe_s = A.rows_total / CS::ROWS;
        plan.shared_mma = false;
        plan.cost_shared = (A.sh_count + CS::TGK - 1) / CS::TGK;
        plan.prefix = s_prefix1;
        const long total = plan.total_cost();
        scur = plan.find(total * blockIdx.x / gridDim.x);
        const Cursor last = plan.find(total * (blockIdx.x + 1) / gridDim.x);
        n_sh = plan.index(last) - plan.index(scur);
    }
    if (DT_S == PMOE_Q8_0 && warp == SHW_WARP) {   // the shared expert's warp
        if (shared_warp) {
            pdl_wait();
            q80_shared_warp<1>(A, lane);
        }
        return;
    }
    if (n_mma + n_sh <= 0) return;

    if (warp == GEMV_WARPS) {   // the producer warp: one lane keeps the ring full
        if (lane != 0 || A.debug == 2) return;
        MmaCursor pc = first;
        int issued = 0;
        bool ok = true;
        for (; issued < n_mma; issued++) {
            const int s = issued % DM_NSTAGE;
            const uint32_t use = (uint32_t)(issued / DM_NSTAGE);
            // the slot must have been released, and its previous copy must have landed: warps that gave up waiting
            // release slots early, and a barrier must not be armed twice in one phase
            if (use > 0 && !(mbar_wait(dm_empty(smem, s), (use - 1) & 1, A.max_polls) &&
                             mbar_wait(dm_full(smem, s), (use - 1) & 1, A.max_polls))) {
                set_status(A.status, PMOE_ERR_TIMEOUT, 33, issued);
                ok = false;
                break;
            }
            const uint8_t *src = (pc.slot < work.n_active ? A.w0 + (size_t)A.g.active[pc.slot] * A.expert_bytes : A.sw0) +
                                 (size_t)pc.chunk * DM_ITEM;
            uint64_t *full = dm_full(smem, s);
            mbar_expect_tx(full, DM_ITEM);
            uint8_t *dst = dm_stage(smem, s);
            for (uint32_t off = 0; off < (uint32_t)DM_ITEM; off += BULK_PIECE)
                bulk_g2s(dst + off, src + off, DM_ITEM - off < (uint32_t)BULK_PIECE ? DM_ITEM - off : (uint32_t)BULK_PIECE, full);
            work.advance(pc);
        }
        if (STREAM_SH && ok && n_sh > 0) {
            // the streaming items reuse the same shared memory: every tensor-core stage must have been
            // released first (which also means its copy has landed)
            for (int it = issued > DM_NSTAGE ? issued - DM_NSTAGE : 0; it < issued && ok; it++)
                if (!mbar_wait(dm_empty(smem, it % DM_NSTAGE), (uint32_t)(it / DM_NSTAGE) & 1, A.max_polls)) {
                    set_status(A.status, PMOE_ERR_TIMEOUT, 34, it);
                    ok = false;
                }
            if (ok) {
                Producer<DT_S1, DT_S1, 1> prod{A, plan, ring2, scur, 0, n_sh};
                for (int i = 0; i < n_sh; i++)
                    if (!prod.issue_next()) { prod.issued--; break; }
                drain_ring(ring2, prod.issued, A.max_polls);
                return;
            }
        }
        // no asynchronous write may reach shared memory after the CTA has left
        for (int it = issued > DM_NSTAGE ? issued - DM_NSTAGE : 0; it < issued; it++)
            mbar_wait(dm_full(smem, it % DM_NSTAGE), (uint32_t)(it / DM_NSTAGE) & 1, A.max_polls);
        return;
    }

    pdl_wait();
    const int team = warp >> 2, mtile = warp & 3;
    bool failed = false;
    {
        MmaCursor cur = first;
        int it = team;
        if (team == 1) work.advance(cur);
        LookAhead la;
        la.slot = la.group = -1;
        la.step = 3;
        while (it < n_mma) {
            const bool is_sh = cur.slot >= work.n_active;
            const int t0 = GEMV_TG_MMA * cur.group;
            int m, my_row = -1;
            if (is_sh) {
                m = A.sh_count;
            } else if (la.ready(work, cur.slot, cur.group)) {
                m = la.m;
                my_row = la.row;
            } else {
                const int e = A.g.active[cur.slot];
                m = A.g.count[e];
                const int i = t0 + (lane & 7);
                if (i < m) my_row = A.g.pairs[A.g.offset[e] + i];
            }
            la.start(cur);
            const int cnt = m - t0 < GEMV_TG_MMA ? m - t0 : GEMV_TG_MMA;
            if (cnt <= 2) dm_run_group<2>(A, smem, work, cur, it, n_mma, is_sh, my_row, t0, cnt, mtile, lane, failed, la);
            else if (cnt <= 4) dm_run_group<4>(A, smem, work, cur, it, n_mma, is_sh, my_row, t0, cnt, mtile, lane, failed, la);
            else dm_run_group<8>(A, smem, work, cur, it, n_mma, is_sh, my_row, t0, cnt, mtile, lane, failed, la);
        }
    }
    if constexpr (STREAM_SH) {
        if (!failed && n_sh > 0) {
            int it = 0;
            run_items<DT_S1, 1>(A, ring2, plan, true, scur, 1, it, n_sh, A.in_s, warp, lane);
        }
    }
}

template <int DT_S> static cudaError_t launch_q6k_mma_t(const GemvArgs &A, cudaStream_t s)
{
    auto kern = k_down_q6k_mma<DT_S>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DM_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaError_t e = launch_pdl(kern, dim3(2 * sm_count()), dim3(DT_S == PMOE_Q8_0 ? SHW_THREADS : GEMV_THREADS), DM_SMEM, s, A);
    count_launch();
    return e;
}

// PMOE_MAX_POLLS in the environment shortens every bounded device-side wait (read at each launch; tests of the
// timeout path use it)
static uint32_t max_polls_env()
{
    const char *e = getenv("PMOE_MAX_POLLS");
    const long v = e ? atol(e) : 0;
    return v > 0 ? (uint32_t)v : (1u << 20);
}

static int shw_min_tokens()
{
    static const int v = getenv("PMOE_SHW_MIN") ? atoi(getenv("PMOE_SHW_MIN")) : 1;
    return v;
}

cudaError_t launch_down_q6k_mma(GemvArgs &A, int dt_s, cudaStream_t s)
{
    A.shw_min = shw_min_tokens();
    A.max_polls = max_polls_env();
    A.stage_bytes = STAGE_BYTES;   // the streaming-kind items of a shared expert of another type
    switch (dt_s) {
    case 0: return launch_q6k_mma_t<0>(A, s);
    case PMOE_Q4_K: return launch_q6k_mma_t<PMOE_Q4_K>(A, s);
    case PMOE_Q5_K: return launch_q6k_mma_t<PMOE_Q5_K>(A, s);
    case PMOE_Q6_K: return launch_q6k_mma_t<PMOE_Q6_K>(A, s);
    case PMOE_Q8_0: return launch_q6k_mma_t<PMOE_Q8_0>(A, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_gate_up_q4k_mma(GemvArgs &A, int dt_s, cudaStream_t s)
{
    A.shw_min = shw_min_tokens();
    A.max_polls = max_polls_env();
    A.stage_bytes = MMA_STAGE_BYTES;
    switch (dt_s) {
    case 0: return launch_q4k_mma_t<0>(A, s);
    case PMOE_Q4_K: return launch_q4k_mma_t<PMOE_Q4_K>(A, s);
    case PMOE_Q5_K: return launch_q4k_mma_t<PMOE_Q5_K>(A, s);
    case PMOE_Q6_K: return launch_q4k_mma_t<PMOE_Q6_K>(A, s);
    case PMOE_Q8_0: return launch_q4k_mma_t<PMOE_Q8_0>(A, s);
    }
    return cudaErrorInvalidValue;
}

// PMOE_MMA in the environment (comparison runs): 0 keeps the dp4a kernels everywhere, 2 takes the tensor-core
// kernel for Q4_K gate/up only, 3 for Q6_K down only; unset or 1: both
bool mma_enabled(int kernel)
{
    static const int mode = getenv("PMOE_MMA") ? atoi(getenv("PMOE_MMA")) : 1;
    return mode == 1 || (mode == 2 && kernel == 1) || (mode == 3 && kernel == 2);
}


}  // namespace pmoe
