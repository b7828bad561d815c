// Batch-1 product straight from the packed tags, by activation-side tables (d = 8, 12-bit tags, 4096-entry books).
//
// For a tile of 8 chunk columns (64 weight columns) a thread block computes the table
//     T[e][c] = <book[e], x_chunk_c>          e = 0..4095, c = 0..7        (mma.sync m16n8k8, 256 per tile)
// once, as 16-bit integers with a power-of-two scale per tile (the scale comes from a Cauchy-Schwarz bound, so no
// entry can saturate), into 64 KB of shared memory; after that every weight chunk (8 weights, 12 bits in HBM)
// costs ONE 2-byte shared-memory read and half an integer add (three-input adds; a row's 8 entries sum exactly).  Two tables
// alternate: while the block looks tile t up, its warps build tile t + 1, so only a block's first build
// is exposed.  The tags of the block's rows stream through a ring of shared-memory stages filled by bulk
// copies (cp.async.bulk + mbarrier, 8 stages = 96 KB in flight, started before the kernel waits for its
// predecessor); nobody is the producer: the last warp to read a stage issues the copies that refill it.  A block owns a rectangle (rows x tiles) of one matrix; a thread owns up to 8 rows
// of it and keeps their fp32 sums in registers over all the block's tiles.
//
// Row sums of blocks that share rows (different tile ranges) meet without atomics, fences or counters, and in a
// FIXED order, so two runs agree bit for bit: every block stores its fp32 partial sums into its own slot of the
// work space as 64-bit words {valid flag, value} (a 64-bit store is indivisible: whoever sees the flag sees the
// value).  Then EVERY block of the row part sums a slice of the part's rows over the splits, in split order -
// polling, with a bound, the words that have not landed yet and clearing each word it has consumed - applies the
// row scale, rounds and writes y.  One kernel per call, the finishing work spread over all SMs, two memory round
// trips after the last lookup.  (All blocks of a launch are resident at once - one block per SM, at most as many
// blocks as SMs - so the poll cannot starve the block it waits for.)
//
// Shared-memory gathers bound this kernel, not HBM: a warp's 32 random 2-byte reads take as many cycles
// as the most loaded bank has requests, 3.3 on average.  Per lane the column it reads rotates with the lane
// index ((slot + row position / 4) mod 8; the tags are stored in that rotated order), which keeps same-column lanes from
// piling on the few banks one column's entries occupy.  A thread takes 4 consecutive rows per step (one 16-byte
// read per tag plane, 32 independent table reads in flight): the loop is bound by latency, not by issue slots.
#include <map>
#include <mutex>
#include <vector>
#include "cbl_common.cuh"


constexpr int L8_NT = 512;                       // threads per block; a thread handles 4 consecutive rows per ring stage
constexpr int L8_NWARP = L8_NT / 32;
constexpr int L8_THREADS = L8_NT;                // the last warp to read a ring stage refills it
constexpr int L8_RPT = 8;                        // rows per thread: a block covers at most 4096 rows
constexpr int L8_STEP_ROWS = 4 * L8_NT;           // 2048 rows per step of the block
constexpr int L8_STAGE_ROWS = L8_STEP_ROWS / 2;   // a ring stage holds half a step: the rows of 8 warps
constexpr int L8_STAGE_WARPS = L8_NWARP / 2;
constexpr int L8_STAGE_BYTES = 3 * L8_STAGE_ROWS * 4;   // three tag planes
constexpr int L8_MAX_STAGES = 8;
constexpr int L8_DYN_SMEM = 231424;              // all of an SM's shared memory but 1 KB for the static part
constexpr int L8_ACC_BYTES = L8_NT * L8_RPT * 4;  // fp32 row sums of a block between tiles
constexpr uint32_t L8_WAIT_LIMIT = 1u << 20;     // mbarrier polls before a wait gives up
constexpr int L8_MAX_GROUP = 4;
constexpr int L8_MAX_BLOCKS = 160;
constexpr int L8_MAX_ORDERS = 16;
constexpr int L8_SLOT_ROWS = L8_NT * L8_RPT;      // partial-sum slot of one block: one 64-bit word per row
constexpr size_t L8_PART_BYTES = (size_t)L8_MAX_BLOCKS * L8_SLOT_ROWS * 8;
constexpr int L8_CTL_WORDS = 64;                 // status word at 0
constexpr int L8_STATUS_WORD = 0;
constexpr uint32_t L8_MEET_LIMIT = 1u << 20;     // polls of another block's partial sums before a block gives up (~1 s)

static inline size_t l8_rows_max(int32_t R) { return ((size_t)R + 31) / 32 * 32 + 32 * L8_MAX_ORDERS; }

// Work space of a launch: partial-sum slots of the blocks | status word | fp32 sums by source row of each
// matrix (mode 1).  The per-matrix figure covers a launch of that matrix alone; a group needs no more than the sum.
extern "C" size_t cbl_gemv_l8_workspace_bytes(int32_t R) {
    if (R < 0) return 0;
    return L8_PART_BYTES + L8_CTL_WORDS * 4 + l8_rows_max(R) * 4;
}

__device__ __forceinline__ void l8_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void l8_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void l8_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// Bounded wait for a phase of an mbarrier; false when the limit ran out.
__device__ __forceinline__ bool l8_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < L8_WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ uint32_t l8_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void l8_sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
// D = A(16x8, row) * B(8x8, col), fp16 inputs, fp32 result; not volatile: the compiler may issue several back to back.
__device__ __forceinline__ void l8_mma1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

// One signed 16-bit table entry (sign-extended) from a shared-memory address.
__device__ __forceinline__ int l8_entry(uint32_t addr) {
    int v;
    asm volatile("ld.shared.s16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Sum of a row's 8 table entries of one tile (exact: the entries are 16-bit integers).  (w0, w1, w2) is the row's
// 96-bit stream of 8 tags, slot s at bit 12 s; col[s] = table base | 2 * column of slot s for this lane.  Entry
// address = base + tag * 16 + column * 2: the base is 64 KB aligned, so the three fields are merged with one logic
// operation per tag.
__device__ __forceinline__ int l8_row8(uint32_t w0, uint32_t w1, uint32_t w2, const uint32_t (&col)[8]) {
    const int e0 = l8_entry(((w0 << 4) & 0xFFF0u) | col[0]);
    const int e1 = l8_entry(((w0 >> 8) & 0xFFF0u) | col[1]);
    const int e2 = l8_entry((__funnelshift_r(w0, w1, 20) & 0xFFF0u) | col[2]);
    const int e3 = l8_entry((w1 & 0xFFF0u) | col[3]);
    const int e4 = l8_entry(((w1 >> 12) & 0xFFF0u) | col[4]);
    const int e5 = l8_entry((__funnelshift_r(w1, w2, 24) & 0xFFF0u) | col[5]);
    const int e6 = l8_entry(((w2 >> 4) & 0xFFF0u) | col[6]);
    const int e7 = l8_entry(((w2 >> 16) & 0xFFF0u) | col[7]);
    return ((e0 + e1) + (e2 + e3)) + ((e4 + e5) + (e6 + e7));
}

// 2^e as a float, e clamped to the normal range.
__device__ __forceinline__ float l8_pow2(int e) {
    e = e < -126 ? -126 : (e > 127 ? 127 : e);
    return __int_as_float((e + 127) << 23);
}

// Power-of-two exponent k such that |v| * 2^-k < 2^14 for the largest magnitude mx (k may be negative).
__device__ __forceinline__ int l8_scale_exp(float mx) {
    if (!(mx > 0.f) || !(mx < 3.0e38f)) return 0;
    int k = ((__float_as_int(mx) >> 23) & 0xFF) - 127 - 13;      // exponent field (subnormals land on the clamp below)
    return k < -100 ? -100 : (k > 110 ? 110 : k);
}

// Up to L8_MAX_GROUP matrices that share one activation vector (q|k|v, gate|up) run as ONE launch.
struct L8Launch {
    int n;                             // matrices in the group
    int ydtype;
    int mode;                          // 0: y = round(row_scale * sum); 1: fsum[source row] = sum (another kernel follows)
    cbl_l8 m[L8_MAX_GROUP];
    unsigned long long* partial;       // L8_MAX_BLOCKS slots of L8_SLOT_ROWS words {valid << 32 | fp32 partial sum} (zero on entry, left zero)
    float* fsum[L8_MAX_GROUP];         // mode 1: fp32 sums by source row
    void* y[L8_MAX_GROUP];
    unsigned int* status;              // set to 1 when a bounded wait expired
    const uint32_t* calls;             // optional: completed-call counter; call e = *calls + 1 writes its sums to
    int64_t fsum_stride;               // fsum[0] + (e & 1) * fsum_stride (two alternating buffers, see cbl_gemv_l8_ar)
};

// One block = one rectangle: rows [row_lo, row_lo + nrows) (positions in the matrix's row order, multiples of
// 32) x tiles [tile_lo, tile_hi) of matrix mi, all rows of one column order.
struct L8Plan {
    int nblocks;
    int4 r[L8_MAX_BLOCKS];   // x = mi | order << 2 | part << 8 | splits << 16 | first block of the part << 24, y = row_lo, z = nrows,
                             // w = tile_lo | tile_hi << 16; the blocks of a part are consecutive, in split order
};

// Barrier among the block's 512 threads.
__device__ __forceinline__ void l8_sync_block() { asm volatile("bar.sync 1, %0;" ::"n"(L8_NT) : "memory"); }

__global__ void __launch_bounds__(L8_THREADS, 1) k_gemv_l8(const __grid_constant__ L8Launch P, const __grid_constant__ L8Plan plan,
                                                           const void* __restrict__ x, int xdtype) {
    extern __shared__ __align__(128) unsigned char l8_smem[];
    __shared__ __align__(8) unsigned long long s_bar[L8_MAX_STAGES];       // full[stage]: the stage's tags have landed
    __shared__ int s_abort;
    __shared__ unsigned int s_readers[L8_MAX_STAGES];   // warps that have read the stage's current contents
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    if ((int)blockIdx.x >= plan.nblocks) return;
    const int4 d = plan.r[blockIdx.x];
    const int mi = d.x & 3, order = (d.x >> 2) & 15, splits = (d.x >> 16) & 255, first = (int)((uint32_t)d.x >> 24);
    const int row_lo = d.y, nrows = d.z, tile_lo = d.w & 0xFFFF, tile_hi = (int)((uint32_t)d.w >> 16);
    const cbl_l8& mm = P.m[mi];
    // Programmatic dependent launch: this kernel waits for its predecessor only where it first touches data that
    // depends on it (x, the work space, y), and lets its successor in when its own lookups are done (below).

    // ---- shared memory: two 64 KB tables on a 64 KB boundary; below and above them the fp32 row sums of the
    // block (16 KB) and the ring stages
    const uint32_t base = cbl_smem_u32(l8_smem), end = base + (uint32_t)L8_DYN_SMEM;
    const uint32_t tbl0 = (base + 65535u) & ~65535u;
    const uint32_t hi0 = tbl0 + 131072u;
    uint32_t lo0 = (base + 127u) & ~127u, hi1 = hi0, sacc;
    if (end >= hi0 + L8_ACC_BYTES) { sacc = hi0; hi1 += L8_ACC_BYTES; } else { sacc = lo0; lo0 += L8_ACC_BYTES; }
    const int n_lo = tbl0 > lo0 ? (int)((tbl0 - lo0) / L8_STAGE_BYTES) : 0;
    const int n_hi = end > hi1 ? (int)((end - hi1) / L8_STAGE_BYTES) : 0;
    const int S = min(L8_MAX_STAGES, n_lo + n_hi);
    if (hi1 > end || S < 2) {                          // cannot happen with the launch configuration of this file
        if (tid == 0) atomicExch(P.status, 2u);
        return;
    }
    auto stage_addr = [&](int s) { return s < n_lo ? lo0 + (uint32_t)s * L8_STAGE_BYTES : hi1 + (uint32_t)(s - n_lo) * L8_STAGE_BYTES; };
    const uint32_t bar0 = cbl_smem_u32(s_bar);

    const int nrow_it = (nrows + L8_STEP_ROWS - 1) / L8_STEP_ROWS;     // <= 2
    const int ntl = tile_hi - tile_lo;
    const int nit = ntl * nrow_it;                     // iterations of this block: (tile, row step), tile-major; two ring stages each
    if (tid < S) {
        l8_mbar_init(bar0 + 8 * tid, 1);                             // full: the issuing lane's arrive + the bytes of three copies
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 0) s_abort = 0;
    if (tid < L8_MAX_STAGES) s_readers[tid] = 0u;
    __syncthreads();

    // ---- tag ring.  Stage n (half n & 1 of iteration n / 2) lives in ring slot n mod S.  Nobody is the producer: the
    // warp that is the LAST of a stage's 8 readers issues the copies of stage n + S into the slot (lanes 0..2 the three
    // tag planes, lane 0 announces the bytes), without waiting for anything.  Weights do not depend on the previous
    // kernel: warp 0 fills the ring before the wait below.
    auto issue = [&](int n) {                           // whole warp; stage n -> slot n mod S
        const int i = n >> 1, ti = i / nrow_it, k = i - ti * nrow_it;
        const int r0 = k * L8_STEP_ROWS + (n & 1) * L8_STAGE_ROWS;
        const int cnt = max(0, min(L8_STAGE_ROWS, nrows - r0));
        const int slot = n % S;
        const uint32_t bar = bar0 + 8 * slot;
        if (lane == 0) {
            if (cnt > 0) l8_mbar_expect_tx(bar, 12u * (uint32_t)cnt);
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");      // an empty half completes at once
        }
        __syncwarp();
        if (lane < 3 && cnt > 0)
            l8_bulk_g2s(stage_addr(slot) + lane * (L8_STAGE_ROWS * 4),
                        (const uint32_t*)mm.words + ((int64_t)(tile_lo + ti) * 3 + lane) * mm.Rpad + row_lo + r0, 4u * (uint32_t)cnt, bar);
    };
    if (warp == 0)
        for (int n = 0; n < S && n < 2 * nit; n++) issue(n);

    // ---- tables.  The book's mma A fragments stay in registers for all tiles of a book (one 16-byte load per two
    // 16-codeword blocks); everything that does not depend on the previous kernel is requested before the wait.
    const int ntile1 = mm.ntile / mm.books;
    uint4 af[8];
    int cur_book = -1, jx = 0;
    auto set_book = [&](int book) {
        const uint4* fr = (const uint4*)(book ? mm.frag2 : mm.frag);
#pragma unroll
        for (int i = 0; i < 8; i++) af[i] = __ldg(fr + (warp + i * L8_NWARP) * 32 + lane);
        // |<codeword, x_chunk>| <= norm * |x_chunk| < 2^(jx + 1) * 2^(13 - jx) = 2^14: every entry fits 16 bits with room to spare
        jx = book ? mm.book_exp2 : mm.book_exp;
        cur_book = book;
    };
    set_book(tile_lo / ntile1);

    asm volatile("griddepcontrol.wait;" ::: "memory");              // x, accumulators and outputs belong to earlier kernels until here
    float* fsum = P.fsum[mi];
    if (P.calls && fsum) fsum += (int64_t)((__ldcg(P.calls) + 1u) & 1u) * P.fsum_stride;

    const int32_t* perm = mm.perms ? mm.perms + (int64_t)order * mm.C : nullptr;
    auto load_x = [&](int tile, float& xa, float& xb) {
        const int ctile = tile % ntile1, c0 = ctile * 64 + 2 * lane;
        xa = xb = 0.f;
        if (c0 < mm.C) {
            xa = cbl_load_in(x, xdtype, perm ? perm[c0] : c0);
            xb = cbl_load_in(x, xdtype, perm ? perm[c0 + 1] : c0 + 1);
        }
    };
    float xa, xb;
    load_x(tile_lo, xa, xb);

    // ---- table build: 16 codeword blocks per warp; the tile's 64 activations are this warp's B fragment
    // (lane (g, t) holds k = 2t, 2t+1 of chunk column g = elements 2 lane, 2 lane + 1 of the tile).  The activations
    // are scaled by a power of two that brings the largest Euclidean norm of the tile's 8 chunks below
    // 2^13 * 2^-jx: the products then stay below 2^14 in magnitude whatever the inputs (Cauchy-Schwarz) and
    // are stored as rounded 16-bit integers; the returned factor undoes the scale on the integer sum of a row.
    auto build = [&](uint32_t tbl, float va, float vb) -> float {
        float me = fmaxf(fabsf(va), fabsf(vb));          // largest element of the tile: a first scale, so that squares cannot overflow
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) me = fmaxf(me, __shfl_xor_sync(0xffffffffu, me, o));
        const int k1 = l8_scale_exp(me);
        const float s1 = l8_pow2(-k1), ua = va * s1, ub = vb * s1;
        float n2 = ua * ua + ub * ub;                    // squared norm of chunk g over its four lanes
        n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
        n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
#pragma unroll
        for (int o = 16; o > 2; o >>= 1) n2 = fmaxf(n2, __shfl_xor_sync(0xffffffffu, n2, o));
        // largest chunk norm -> [2^12, 2^13) * 2^-jx: one bit of head room for the rounding of the fp16 activations
        // (floor(log2(sqrt(n2))) is half the exponent of n2, which is at least 2^26 here)
        const int k2 = n2 > 0.f ? ((((__float_as_int(n2) >> 23) & 0xFF) - 127) >> 1) - 12 : 0;
        const int k = k1 + (k2 > 0 ? k2 : 0) + jx;
        // a NaN or infinity among the tile's activations must reach every output, as it would in a matrix product
        const bool nonfinite = __any_sync(0xffffffffu, !(fabsf(va) <= 3.0e38f) || !(fabsf(vb) <= 3.0e38f));
        const float sc = l8_pow2(-k);
        const __half2 xh = __floats2half2_rn(va * sc, vb * sc);
        const uint32_t b0 = *(const uint32_t*)&xh;
        const uint32_t a0 = tbl + (uint32_t)g * 16u + (uint32_t)t * 4u + (uint32_t)warp * 512u;
        // four products in flight at a time (their latencies overlap), then the eight stores of the group
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float c[4][4];
            l8_mma1688(c[0], af[i].x, af[i].y, b0);
            l8_mma1688(c[1], af[i].z, af[i].w, b0);
            l8_mma1688(c[2], af[i + 1].x, af[i + 1].y, b0);
            l8_mma1688(c[3], af[i + 1].z, af[i + 1].w, b0);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                // round to integer by adding 1.5 * 2^23: the low 16 bits of the sum's pattern are the two's-complement value
                const uint32_t lo = __byte_perm(__float_as_uint(c[q][0] + 12582912.f), __float_as_uint(c[q][1] + 12582912.f), 0x5410);
                const uint32_t hi = __byte_perm(__float_as_uint(c[q][2] + 12582912.f), __float_as_uint(c[q][3] + 12582912.f), 0x5410);
                const uint32_t a = a0 + (uint32_t)((i + (q >> 1)) * L8_NWARP * 512 + (q & 1) * 256);   // codeword block ((warp + 16 i') * 2 + h) * 16
                l8_sts32(a, lo);
                l8_sts32(a + 128u, hi);
            }
        }
        return nonfinite ? __int_as_float(0x7fc00000) : l8_pow2(k);
    };

    uint32_t col[8];
#pragma unroll
    for (int s = 0; s < 8; s++) col[s] = tbl0 | (uint32_t)(((s + lane) & 7) << 1);

    float inv_cur = build(tbl0, xa, xb), inv_nxt = 0.f;
    if (ntl > 1) load_x(tile_lo + 1, xa, xb);

    l8_sync_block();                                // the first table is complete

    // ---- main loop over the ring iterations.  Warps run through the ring on their own; the tags of iteration i + 1
    // are fetched from the ring before the lookups of iteration i; a row's fp32 sum lives in shared memory between
    // tiles (each row belongs to one thread).  After a wait has expired the loop only keeps its shape (it contains
    // barriers) and does no more work.
    const int half = warp / L8_STAGE_WARPS, tih = tid - half * (L8_NT / 2);    // this thread's half step and index in it
    int cstage = half, kf = 0, cn = half;              // ring slot, row step and stage number of the next fetch
    uint32_t cphase = 0;
    bool dead = false;
    uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0, w2 = w0;
    auto fetch = [&]() {                                // tags of the next ring iteration (row step kf) -> w0..w2
        if (!dead && !l8_mbar_wait(bar0 + 8 * cstage, cphase)) { s_abort = 1; dead = true; }
        w0 = w1 = w2 = make_uint4(0, 0, 0, 0);
        if (!dead && kf * L8_STEP_ROWS + 4 * tid < nrows) {
            const uint32_t a = stage_addr(cstage) + (uint32_t)tih * 16u;
            w0 = cbl_lds128(a);
            w1 = cbl_lds128(a + L8_STAGE_ROWS * 4);
            w2 = cbl_lds128(a + 2 * L8_STAGE_ROWS * 4);
        }
        __syncwarp();
        // the last of the stage's readers refills its slot with the stage S further on
        unsigned int last = 0;
        if (lane == 0 && atomicAdd(&s_readers[cstage], 1u) == L8_STAGE_WARPS - 1) {
            atomicExch(&s_readers[cstage], 0u);
            last = 1;
        }
        if (__shfl_sync(0xffffffffu, last, 0) && cn + S < 2 * nit && !dead) issue(cn + S);
        cn += 2;
        cstage += 2;
        if (cstage >= S) { cstage -= S; cphase ^= 1u; }
        if (++kf == nrow_it) kf = 0;
    };
    fetch();
    float acc[2][4];                                    // this thread's 4 rows of row step 0 and of row step 1
#pragma unroll
    for (int u = 0; u < 4; u++) acc[0][u] = acc[1][u] = 0.f;
    int k = 0, ti = 0;
    for (int it = 0; it < nit; it++) {
        // The next tile's table goes into the other buffer while this tile is looked up: one half of the warps builds
        // its share before its lookups of the tile, the other half after them, so that at any time some warps keep the
        // shared-memory pipe busy with lookups while others run the tensor-core products of the build.
        const bool build_now = ti + 1 < ntl && (half == 0 ? k == 0 : k == nrow_it - 1);
        if (build_now && half == 0) {
            const int nb = (tile_lo + ti + 1) / ntile1;
            if (nb != cur_book) set_book(nb);
            inv_nxt = build(tbl0 + (uint32_t)(((ti + 1) & 1) << 16), xa, xb);
            if (ti + 2 < ntl) load_x(tile_lo + ti + 2, xa, xb);
        }
        const uint4 c0 = w0, c1 = w1, c2 = w2;
        dead = dead || *(volatile int*)&s_abort != 0;
        const bool act = !dead && k * L8_STEP_ROWS + 4 * tid < nrows;
        if (it + 1 < nit) fetch();
        if (act) {
            const float r0 = (float)l8_row8(c0.x, c1.x, c2.x, col) * inv_cur, r1 = (float)l8_row8(c0.y, c1.y, c2.y, col) * inv_cur;
            const float r2 = (float)l8_row8(c0.z, c1.z, c2.z, col) * inv_cur, r3 = (float)l8_row8(c0.w, c1.w, c2.w, col) * inv_cur;
            if (k == 0) { acc[0][0] += r0; acc[0][1] += r1; acc[0][2] += r2; acc[0][3] += r3; }
            else { acc[1][0] += r0; acc[1][1] += r1; acc[1][2] += r2; acc[1][3] += r3; }
        }
        if (build_now && half == 1) {
            const int nb = (tile_lo + ti + 1) / ntile1;
            if (nb != cur_book) set_book(nb);
            inv_nxt = build(tbl0 + (uint32_t)(((ti + 1) & 1) << 16), xa, xb);
            if (ti + 2 < ntl) load_x(tile_lo + ti + 2, xa, xb);
        }
        if (++k == nrow_it) {
            k = 0;
            ti++;
            const uint32_t tn = tbl0 + (uint32_t)((ti & 1) << 16);
#pragma unroll
            for (int s = 0; s < 8; s++) col[s] = (col[s] & 0xFFFFu) | tn;
            inv_cur = inv_nxt;
            l8_sync_block();                        // next table complete; every reader of this one is done
        }
    }
    // The next kernel of the stream may become resident from here on.  (Not earlier: a block of this kernel fills its
    // SM, so an early successor would be packed onto the few SMs this launch leaves free instead of spreading
    // over the SMs as they empty.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the row sums go to shared memory, indexed by row of the block, for the output phase
#pragma unroll
    for (int kk = 0; kk < 2; kk++)
        if (kk * L8_STEP_ROWS + 4 * tid < nrows)
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(sacc + (uint32_t)(kk * L8_STEP_ROWS + 4 * tid) * 4u), "f"(acc[kk][0]),
                         "f"(acc[kk][1]), "f"(acc[kk][2]), "f"(acc[kk][3])
                         : "memory");
    l8_sync_block();
    if (*(volatile int*)&s_abort) {
        // a staged copy never completed: report and leave (the waits that gave up were bounded)
        if (tid == 0) atomicExch(P.status, 1u);
        return;
    }

    // ---- row sums -> outputs
    const int32_t* rix = mm.row_index;
    auto source_row = [&](int p) {                      // source row of row position p, -1 for padding
        const int r = rix ? rix[p] : p;
        return r < mm.R ? r : -1;
    };
    auto emit = [&](int r, float v) {
        if (P.mode == 0) cbl_store_out(P.y[mi], P.ydtype, r, v * __half2float(((const __half*)mm.row_scale)[r]));
        else fsum[r] = v;
    };
    const int n512 = (nrows + L8_NT - 1) / L8_NT;
    if (splits <= 1) {
        for (int j = 0; j < n512; j++) {
            const int q = j * L8_NT + tid;
            if (q >= nrows) break;
            const int r = source_row(row_lo + q);
            if (r >= 0) emit(r, __uint_as_float(l8_lds32(sacc + (uint32_t)q * 4u)));
        }
        return;
    }
    // this block's partial sums -> its slot, each with its valid flag
    unsigned long long* slot = P.partial + (size_t)blockIdx.x * L8_SLOT_ROWS;
    for (int j = 0; j < n512; j++) {
        const int q = j * L8_NT + tid;
        if (q < nrows) __stcg(slot + q, (1ull << 32) | (unsigned long long)l8_lds32(sacc + (uint32_t)q * 4u));
    }
    l8_sync_block();                                // the row sums in shared memory have been read: the space is staging now
    // every block sums its share of the part's rows over the splits: thread (row, group) adds the splits
    // group, group + G, ... in order, the groups are added in order through shared memory
    const int s_me = (int)blockIdx.x - first;
    const int q_lo = (int)((int64_t)nrows * s_me / splits), q_hi = (int)((int64_t)nrows * (s_me + 1) / splits);
    const int nq = q_hi - q_lo;
    unsigned long long* slots = P.partial + (size_t)first * L8_SLOT_ROWS;
    bool late = false;
    for (int q0 = 0; q0 < nq; q0 += L8_NT) {
        const int nqq = min(L8_NT, nq - q0);
        int G = L8_NT / nqq;
        if (G > splits) G = splits;
        const int r = tid % nqq, grp = tid / nqq;
        // the output row and its scale are requested before the partial sums, not after them
        int rr = -1;
        float rsc = 0.f;
        if (grp == 0) {
            rr = source_row(row_lo + q_lo + q0 + r);
            if (rr >= 0 && P.mode == 0) rsc = __half2float(((const __half*)mm.row_scale)[rr]);
        }
        float sum = 0.f;
        if (grp < G) {
            unsigned long long* src = slots + q_lo + q0 + r;
            for (int j0 = grp; j0 < splits; j0 += 8 * G) {
                float v[8];
                uint32_t need = 0;
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (j0 + u * G < splits) need |= 1u << u;
                for (uint32_t poll = 0; need && poll < L8_MEET_LIMIT; poll++) {
                    unsigned long long w[8];
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        if (need >> u & 1u) asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[u]) : "l"(src + (size_t)(j0 + u * G) * L8_SLOT_ROWS) : "memory");
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        if ((need >> u & 1u) && (w[u] >> 32)) {
                            v[u] = __uint_as_float((uint32_t)w[u]);
                            need &= ~(1u << u);
                            __stcg(src + (size_t)(j0 + u * G) * L8_SLOT_ROWS, 0ull);     // consumed: clear it for the next call
                        }
                }
                if (need) late = true;
#pragma unroll
                for (int u = 0; u < 8; u++)
                    if (j0 + u * G < splits) sum += v[u];
            }
        }
        if (G > 1) {
            l8_sync_block();                        // previous readers of the staging rows
            if (grp < G) l8_sts32(sacc + (uint32_t)(grp * nqq + r) * 4u, __float_as_uint(sum));
            l8_sync_block();
            if (grp == 0) {
                sum = 0.f;
                for (int gq = 0; gq < G; gq++) sum += __uint_as_float(l8_lds32(sacc + (uint32_t)(gq * nqq + r) * 4u));
            }
        }
        if (grp == 0 && rr >= 0 && !late) {
            if (P.mode == 0) cbl_store_out(P.y[mi], P.ydtype, rr, sum * rsc);
            else fsum[rr] = sum;
        }
    }
    if (late) atomicExch(P.status, 3u);                 // another block's sums never came (cannot happen while all blocks are resident)
}

// ------------------------------------------------------------------------------------ work split (host)
//
// Every (matrix, column order) with rows is cut into row parts x tile splits; a block takes one rectangle.
// The cut minimises the slowest block under a cost model in clock cycles: a table build costs L8_COST_BUILD,
// the lookups of a tile L8_COST_ROW per row (the shared-memory pipe is the bound) but at least L8_COST_MIN.
constexpr double L8_COST_BUILD = 650.0, L8_COST_ROW = 1.0, L8_COST_MIN = 300.0;

struct L8Seg { int mi, order, row0, nrows, ntile; };

static inline double l8_tile_cost(int rows) {
    const double lk = L8_COST_ROW * rows;
    return L8_COST_BUILD + (lk > L8_COST_MIN ? lk : L8_COST_MIN);
}

// Fewest blocks that finish segment s within T; 0 if impossible.  Rows are handled in units of 32.
static int l8_seg_blocks(const L8Seg& s, double T, int* pr_out, int* ks_out) {
    const int u = s.nrows / 32;
    int best = 0;
    const int pr_min = (s.nrows + L8_NT * L8_RPT - 1) / (L8_NT * L8_RPT);
    for (int pr = pr_min; pr <= u && pr <= L8_MAX_BLOCKS; pr++) {
        const int rows = (u + pr - 1) / pr * 32;
        const int tpb = (int)(T / l8_tile_cost(rows));
        if (tpb < 1) continue;
        const int ks = (s.ntile + tpb - 1) / tpb;
        if (ks > 255) continue;
        if (!best || pr * ks < best) { best = pr * ks; *pr_out = pr; *ks_out = ks; }
    }
    return best;
}

static int l8_make_plan(const std::vector<L8Seg>& segs, int maxb, L8Plan* plan) {
    double lo = 0.0, hi = 0.0;
    for (const L8Seg& s : segs) {
        const int rows = s.nrows < L8_NT * L8_RPT ? s.nrows : L8_NT * L8_RPT;
        const double c = s.ntile * l8_tile_cost(rows);
        if (c > hi) hi = c;
    }
    auto total = [&](double T) {
        int sum = 0, pr, ks;
        for (const L8Seg& s : segs) {
            const int b = l8_seg_blocks(s, T, &pr, &ks);
            if (!b) return maxb + 1;
            sum += b;
        }
        return sum;
    };
    if (total(hi) > maxb) return CBL_EUNSUPPORTED;       // more (matrix, column order) pairs than blocks
    for (int it = 0; it < 48 && hi - lo > 1.0; it++) {
        const double mid = 0.5 * (lo + hi);
        if (total(mid) <= maxb) hi = mid; else lo = mid;
    }
    int nb = 0, part = 0;
    for (const L8Seg& s : segs) {
        int pr = 1, ks = 1;
        l8_seg_blocks(s, hi, &pr, &ks);
        const int u = s.nrows / 32;
        if (ks > s.ntile) ks = s.ntile;
        if (pr > u) pr = u;
        for (int p = 0; p < pr; p++) {
            const int u0 = (int)((int64_t)u * p / pr), u1 = (int)((int64_t)u * (p + 1) / pr);
            const int first = nb;
            for (int k = 0; k < ks; k++) {
                const int t0 = (int)((int64_t)s.ntile * k / ks), t1 = (int)((int64_t)s.ntile * (k + 1) / ks);
                plan->r[nb++] = make_int4(s.mi | (s.order << 2) | (part << 8) | (ks << 16) | (first << 24), s.row0 + u0 * 32, (u1 - u0) * 32,
                                          t0 | (t1 << 16));
            }
            part++;
        }
    }
    plan->nblocks = nb;
    return CBL_OK;
}

// ------------------------------------------------------------------------------------ book and tag re-layouts
//
// Book in mma.m16n8k8 A-fragment order: uint4 [128][32] = {a0, a1 of codeword block 2p, a0, a1 of block 2p+1}
// for lane (g, t): a0 = codeword (16*blk + g) values 2t, 2t+1; a1 = codeword (16*blk + g + 8) values 2t, 2t+1;
// followed by two floats: the largest |value| of the book and the largest Euclidean norm of a codeword (rounded up;
// it bounds every table entry).
__global__ void __launch_bounds__(256) k_repack_book(const uint32_t* __restrict__ table, uint4* __restrict__ out, unsigned int* __restrict__ maxbits) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;       // 0 .. 4095
    const int lane = i & 31, p = i >> 5, g = lane >> 2, t = lane & 3;
    uint4 v;
    v.x = table[((2 * p) * 16 + g) * 4 + t];
    v.y = table[((2 * p) * 16 + g + 8) * 4 + t];
    v.z = table[((2 * p + 1) * 16 + g) * 4 + t];
    v.w = table[((2 * p + 1) * 16 + g + 8) * 4 + t];
    out[i] = v;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float m = 0.f, nrm = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 f = __half22float2(*(const __half2*)&w[k]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));             // NaN entries are ignored, infinities kept
        float q = f.x * f.x + f.y * f.y;                         // this lane's quarter of one codeword's squared norm
        q += __shfl_xor_sync(0xffffffffu, q, 1);
        q += __shfl_xor_sync(0xffffffffu, q, 2);
        nrm = fmaxf(nrm, q);
    }
    nrm = sqrtf(nrm) * 1.0001f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        nrm = fmaxf(nrm, __shfl_xor_sync(0xffffffffu, nrm, o));
    }
    if (lane == 0) {
        atomicMax(maxbits, __float_as_uint(m));                  // non-negative floats order like their bit patterns
        atomicMax(maxbits + 1, __float_as_uint(nrm));
    }
}

extern "C" size_t cbl_book_frag_bytes(void) { return 65536 + 16; }

extern "C" int cbl_book_norm_exp(const void* frag, int32_t* exp_out, cbl_stream s) {
    if (!frag || !exp_out) return CBL_EINVAL;
    float nb = 0.f;
    CBL_CUDA(cudaMemcpyAsync(&nb, (const char*)frag + 65536 + 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    CBL_CUDA(cudaStreamSynchronize((cudaStream_t)s));
    int e = (nb > 0.f && nb < 3.0e38f) ? ilogbf(nb) : 0;
    *exp_out = e < -8 ? -8 : (e > 24 ? 24 : e);
    return CBL_OK;
}

extern "C" int cbl_repack_book(const void* table, void* out, cbl_stream s) {
    if (!table || !out || ((uintptr_t)table % 4) || ((uintptr_t)out % 16)) return CBL_EINVAL;
    CBL_CUDA(cudaMemsetAsync((char*)out + 65536, 0, 16, (cudaStream_t)s));
    k_repack_book<<<16, 256, 0, (cudaStream_t)s>>>((const uint32_t*)table, (uint4*)out, (unsigned int*)((char*)out + 65536));
    return cbl_check_launch();
}

// Rotated column-tile layout: uint32 [ntile][3][Rpad].  Position p of the row order holds source row row_index[p]
// (or p itself when row_index is NULL; -1 and p >= R are padding rows of zero tags).  The 8 tags of a row and tile
// form a 96-bit stream whose slot s holds chunk column (s + p / 4) mod 8; word k of that stream is stored at [tile][k][p].
extern "C" size_t cbl_l8r_bytes(int32_t Rpad, int32_t C, int32_t books) {
    if (Rpad < 0 || C <= 0 || books < 1) return 0;
    return (size_t)books * cbl_ceil_div(C / 8, 8) * 3 * (size_t)Rpad * 4;
}

__global__ void __launch_bounds__(256) k_repack_l8r(cbl_packed m, const int32_t* __restrict__ row_index, int ntile1, int Rpad,
                                                    uint32_t* __restrict__ out, int64_t nthreads) {
    const int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= nthreads) return;
    const int p = (int)(gi % Rpad), v = (int)(gi / Rpad);
    const int book = v / ntile1, tile = v % ntile1;
    const int nch = m.C / 8;
    const int32_t* words = book ? m.tags2 : m.tags;
    int r = row_index ? row_index[p] : p;
    if (r >= m.R) r = -1;
    uint32_t w[4] = {0, 0, 0, 0};
    if (r >= 0) {
#pragma unroll
        for (int s = 0; s < 8; s++) {
            const int chunk = tile * 8 + ((s + (p >> 2)) & 7);
            const uint32_t tag = chunk < nch ? cbl_read_tag(words + (int64_t)r * m.W, m.W, chunk, 12) : 0u;
            const int bit = 12 * s;
            w[bit >> 5] |= tag << (bit & 31);
            if ((bit & 31) > 20) w[(bit >> 5) + 1] |= tag >> (32 - (bit & 31));
        }
    }
    uint32_t* o = out + (int64_t)v * 3 * Rpad + p;
    o[0] = w[0];
    o[Rpad] = w[1];
    o[2 * (int64_t)Rpad] = w[2];
}

extern "C" int cbl_repack_l8r(const cbl_packed* m, const int32_t* row_index, int32_t Rpad, void* out, cbl_stream s) {
    if (!m || !m->tags || !m->table || !m->row_scale || !out || ((uintptr_t)out % 16)) return CBL_EINVAL;
    if (m->d != 8 || m->bits != 12 || m->G != 1) return CBL_EUNSUPPORTED;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->tags2) return CBL_EINVAL;
    if (m->R < 0 || m->C <= 0 || m->C % 8 || Rpad < 0 || Rpad % 32) return CBL_EINVAL;
    if (!row_index && Rpad < m->R) return CBL_EINVAL;
    if ((int64_t)m->W * 32 < (int64_t)(m->C / 8) * 12) return CBL_EINVAL;
    const int ntile1 = cbl_ceil_div(m->C / 8, 8);
    const int64_t n = (int64_t)m->books * ntile1 * Rpad;
    if (n == 0) return CBL_OK;
    k_repack_l8r<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)s>>>(*m, row_index, ntile1, Rpad, (uint32_t*)out, n);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ launch
static int check_l8r(const cbl_l8* m) {
    if (!m || !m->words || !m->frag || !m->row_scale) return CBL_EINVAL;
    if (m->rot != 1) return CBL_EINVAL;                          // the product reads the rotated layout only
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->frag2) return CBL_EINVAL;
    if (m->R < 0 || m->C <= 0 || m->C % 8 || m->Rpad < 0 || m->Rpad % 32) return CBL_EINVAL;
    if (m->ntile != m->books * cbl_ceil_div(m->C / 8, 8) || m->ntile >= 65536) return CBL_EINVAL;
    if (m->M < 1 || m->M > L8_MAX_ORDERS) return CBL_EUNSUPPORTED;
    if (m->M > 1 && (!m->perms || !m->row_index)) return CBL_EINVAL;
    if (m->book_exp < -8 || m->book_exp > 24 || (m->books == 2 && (m->book_exp2 < -8 || m->book_exp2 > 24))) return CBL_EINVAL;
    if (!m->row_index && m->Rpad < m->R) return CBL_EINVAL;
    if ((size_t)m->Rpad > l8_rows_max(m->R)) return CBL_EINVAL;
    if (m->seg_off[0] != 0 || m->seg_off[m->M] != m->Rpad) return CBL_EINVAL;
    for (int i = 0; i < m->M; i++)
        if (m->seg_off[i + 1] < m->seg_off[i] || m->seg_off[i] % 32) return CBL_EINVAL;
    if (((uintptr_t)m->words % 16) || ((uintptr_t)m->frag % 16)) return CBL_EINVAL;
    if (m->books == 2 && ((uintptr_t)m->frag2 % 16)) return CBL_EINVAL;
    return CBL_OK;
}

static void l8_segments(const cbl_l8* mats, int n, std::vector<L8Seg>& segs) {
    for (int i = 0; i < n; i++)
        for (int o = 0; o < mats[i].M; o++) {
            const int rows = mats[i].seg_off[o + 1] - mats[i].seg_off[o];
            if (rows > 0) segs.push_back({i, o, mats[i].seg_off[o], rows, mats[i].ntile});
        }
}

// The work split of a group as the launch would make it, for inspection on the host (no device needed):
// out[8 * b .. 8 * b + 7] = {matrix, column order, row part, tile splits of the part, first row position, rows,
// first tile, end tile} of block b; *nblocks = blocks used (at most max_blocks <= 160).
extern "C" int cbl_gemv_l8_plan(const cbl_l8* mats, int32_t n, int32_t max_blocks, int32_t* out, int32_t* nblocks) {
    if (!mats || !out || !nblocks || n < 1 || max_blocks < 1) return CBL_EINVAL;
    if (n > L8_MAX_GROUP) return CBL_EUNSUPPORTED;
    if (max_blocks > L8_MAX_BLOCKS) max_blocks = L8_MAX_BLOCKS;
    std::vector<L8Seg> segs;
    for (int i = 0; i < n; i++) {
        const cbl_l8* m = mats + i;
        if (m->rot != 1 || m->M < 1 || m->M > L8_MAX_ORDERS || m->ntile < 1 || m->ntile >= 65536 || m->Rpad % 32) return CBL_EINVAL;
        for (int o = 0; o < m->M; o++)
            if (m->seg_off[o + 1] < m->seg_off[o] || m->seg_off[o] % 32 || m->seg_off[o + 1] % 32) return CBL_EINVAL;
    }
    l8_segments(mats, n, segs);
    L8Plan plan;
    plan.nblocks = 0;
    if (!segs.empty()) {
        int rc = l8_make_plan(segs, max_blocks, &plan);
        if (rc) return rc;
    }
    for (int b = 0; b < plan.nblocks; b++) {
        const int4 d = plan.r[b];
        int32_t* o = out + 8 * b;
        o[0] = d.x & 3; o[1] = (d.x >> 2) & 15; o[2] = (d.x >> 8) & 255; o[3] = (d.x >> 16) & 255;
        o[4] = d.y; o[5] = d.z; o[6] = d.w & 0xFFFF; o[7] = (int)((uint32_t)d.w >> 16);
    }
    *nblocks = plan.nblocks;
    return CBL_OK;
}

static int launch_l8(L8Launch& P, const void* x, int xdtype, cudaStream_t st, int max_blocks = L8_MAX_BLOCKS, L8Plan* plan_out = nullptr) {
    static bool attr_set[64] = {};
    static std::mutex mu;
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CBL_EUNSUPPORTED;
    int grid = cbl_sm_count();                          // one block per SM: every block of the launch is resident at once
    if (grid > max_blocks) grid = max_blocks;
    // plan cache: the cut depends only on the shapes of the group
    static std::map<std::vector<int>, L8Plan> cache;
    std::vector<int> key = {grid, P.n};
    for (int i = 0; i < P.n; i++) {
        key.push_back(P.m[i].ntile);
        key.push_back(P.m[i].M);
        for (int o = 0; o <= P.m[i].M; o++) key.push_back(P.m[i].seg_off[o]);
    }
    L8Plan plan;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            CBL_CUDA(cudaFuncSetAttribute(k_gemv_l8, cudaFuncAttributeMaxDynamicSharedMemorySize, L8_DYN_SMEM));
            attr_set[dev] = true;
        }
        auto it = cache.find(key);
        if (it == cache.end()) {
            std::vector<L8Seg> segs;
            l8_segments(P.m, P.n, segs);
            plan.nblocks = 0;
            int rc = segs.empty() ? CBL_OK : l8_make_plan(segs, grid, &plan);
            if (rc) return rc;
            cache.emplace(key, plan);
        } else plan = it->second;
    }
    if (plan_out) *plan_out = plan;
    if (plan.nblocks == 0) return CBL_OK;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(plan.nblocks);
    cfg.blockDim = dim3(L8_THREADS);
    cfg.dynamicSmemBytes = L8_DYN_SMEM;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_l8, P, plan, x, xdtype));
    return cbl_check_launch();
}

// Fills the launch descriptor of a group.  Work space: partial-sum slots | status word | fp32 sums of matrix 0,
// matrix 1, ... (l8_rows_max(R_i) floats each).
static int l8_group(const cbl_l8* mats, int32_t n, const void* x, int xdtype, void* const* ys, int ydtype, int mode, void* workspace,
                    L8Launch& P) {
    if (!mats || !x || !workspace || n < 1) return CBL_EINVAL;
    if (n > L8_MAX_GROUP) return CBL_EUNSUPPORTED;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if ((uintptr_t)workspace % 16) return CBL_EINVAL;
    P.n = 0;
    P.ydtype = ydtype;
    P.mode = mode;
    P.partial = (unsigned long long*)workspace;
    P.status = (unsigned int*)((char*)workspace + L8_PART_BYTES) + L8_STATUS_WORD;
    size_t off = L8_PART_BYTES + L8_CTL_WORDS * 4;
    for (int i = 0; i < n; i++) {
        int rc = check_l8r(mats + i);
        if (rc) return rc;
        if (mats[i].C != mats[0].C) return CBL_EINVAL;          // one shared activation vector
        if (ys && !ys[i]) return CBL_EINVAL;
        char* reg = (char*)workspace + off;
        off += l8_rows_max(mats[i].R) * 4;
        if (mats[i].R == 0) continue;
        P.m[P.n] = mats[i];
        P.fsum[P.n] = (float*)reg;
        P.y[P.n] = ys ? ys[i] : nullptr;
        P.n++;
    }
    P.calls = nullptr;
    P.fsum_stride = 0;
    return CBL_OK;
}

extern "C" int cbl_gemv_l8_multi(const cbl_l8* mats, int32_t n, const void* x, int xdtype, void* const* ys, int ydtype,
                                 void* workspace, cbl_stream s) {
    if (!ys) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    L8Launch P;
    int rc = l8_group(mats, n, x, xdtype, ys, ydtype, 0, workspace, P);
    if (rc) return rc;
    if (P.n == 0) return CBL_OK;
    return launch_l8(P, x, xdtype, (cudaStream_t)s);
}

extern "C" int cbl_gemv_l8(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* workspace, cbl_stream s) {
    if (!m || !y) return CBL_EINVAL;
    void* ys[1] = {y};
    return cbl_gemv_l8_multi(m, 1, x, xdtype, ys, ydtype, workspace, s);
}

// Reads and clears the status word a product leaves in its work space (0 = ok, nonzero = a bounded device-side
// wait expired and the output is invalid).  Synchronises the stream.
extern "C" int cbl_gemv_l8_status(void* workspace, int32_t R, cbl_stream s) {
    if (!workspace || R < 0) return CBL_EINVAL;
    char* p = (char*)workspace + L8_PART_BYTES + L8_STATUS_WORD * 4;
    unsigned int v = 0;
    CBL_CUDA(cudaMemcpyAsync(&v, p, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    CBL_CUDA(cudaStreamSynchronize((cudaStream_t)s));
    if (v) CBL_CUDA(cudaMemsetAsync(workspace, 0, L8_PART_BYTES + L8_CTL_WORDS * 4, (cudaStream_t)s));   // and whatever the slots still hold
    return v ? CBL_ETIMEOUT : CBL_OK;
}

// ------------------------------------------------------------------------------------ batch-1 products with a decode-step epilogue
//
// In a decode step most products are followed by a small operator on their output vector.  These entry
// points run that operator in a small second kernel on the fp32 sums (no round trip of the rounded vector
// through memory and one launch less than product + operator); results are identical to the separate
// operators of the step library because the product is rounded to the model's 16-bit type first, exactly
// as if it had been stored.
//   gate|up  -> silu(gate) * up                      (cbl_silu_mul)
//   o / down -> residual add + RMSNorm               (cbl_add_rmsnorm): the kernel's blocks form one
//               cluster and exchange their sums of squares through distributed shared memory
//   q|k|v    -> bias, rotary embedding, cache write  (cbl_rope_kv, decode form, sequence 0)
template <typename T> __device__ __forceinline__ float l8_f(T v);
template <> __device__ __forceinline__ float l8_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float l8_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void l8_pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(256) k_l8_finish_silu(const __grid_constant__ L8Launch P, T* __restrict__ out) {
    l8_pdl_enter();
    const cbl_l8& mg = P.m[0];
    const cbl_l8& mu = P.m[1];
    const int gi = blockIdx.x * blockDim.x + threadIdx.x;
    if (gi * 4 >= mg.R) return;
    const float4 g = __ldcg((const float4*)P.fsum[0] + gi), u = __ldcg((const float4*)P.fsum[1] + gi);
    const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int r = gi * 4 + k;
        if (r < mg.R) {
            const T ga = cbl_cvt_out<T>(gv[k] * __half2float(((const __half*)mg.row_scale)[r]));
            const T ub = cbl_cvt_out<T>(uv[k] * __half2float(((const __half*)mu.row_scale)[r]));
            if (P.y[0]) ((T*)P.y[0])[r] = ga;            // the products themselves, when the caller wants them too
            if (P.y[1]) ((T*)P.y[1])[r] = ub;
            const float a = l8_f(ga), b = l8_f(ub);
            const float sl = l8_f(cbl_cvt_out<T>(a / (1.f + __expf(-a))));
            out[r] = cbl_cvt_out<T>(sl * b);
        }
    }
}

constexpr int L8_NORM_MAX_CTAS = 8;          // portable cluster size: up to 8 x 1024 rows
template <typename T>
__global__ void __launch_bounds__(256) k_l8_finish_addnorm(const __grid_constant__ L8Launch P,
                                                           float* __restrict__ h, const T* __restrict__ w, float eps, T* __restrict__ xout) {
    l8_pdl_enter();
    __shared__ float s_warp[8];
    __shared__ float s_ss, s_tot;
    const cbl_l8& mm = P.m[0];
    const int tid = threadIdx.x, gi = blockIdx.x * blockDim.x + tid, nb = gridDim.x;
    float hv[4] = {0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
    if (gi * 4 < mm.R) {
        const float4 v = __ldcg((const float4*)P.fsum[0] + gi);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int r = gi * 4 + k;
            if (r < mm.R) {
                const T yv = cbl_cvt_out<T>(vv[k] * __half2float(((const __half*)mm.row_scale)[r]));
                if (P.y[0]) ((T*)P.y[0])[r] = yv;        // the product itself, when the caller wants it too
                hv[k] = h[r] + l8_f(yv);
                h[r] = hv[k];
                ss += hv[k] * hv[k];
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) s_warp[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) s_ss = ((s_warp[0] + s_warp[1]) + (s_warp[2] + s_warp[3])) + ((s_warp[4] + s_warp[5]) + (s_warp[6] + s_warp[7]));
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < 32) {
        float v = 0.f;
        if (tid < nb) {
            uint32_t a;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(cbl_smem_u32(&s_ss)), "r"(tid));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
        }
        // fixed order of addition over the blocks: every block computes the same total
        float tot = 0.f;
        for (int k = 0; k < nb; k++) tot += __shfl_sync(0xffffffffu, v, k);
        if (tid == 0) s_tot = tot;
    }
    __syncthreads();
    const float rstd = rsqrtf(s_tot / (float)mm.R + eps);
    if (gi * 4 < mm.R) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int r = gi * 4 + k;
            if (r < mm.R) xout[r] = cbl_cvt_out<T>(hv[k] * rstd * l8_f(w[r]));
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");      // no block leaves while another may still read its sum
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(64) k_l8_finish_rope(const __grid_constant__ L8Launch P, const T* __restrict__ bias,
                                                       const int32_t* __restrict__ pos, int NH, int NKV, int HD, float theta, int max_len,
                                                       T* __restrict__ qo, T* __restrict__ kc, T* __restrict__ vc) {
    l8_pdl_enter();
    const int hd = blockIdx.x, i = threadIdx.x, half = HD >> 1;
    if (i >= half) return;
    const int p = pos[0];
    const bool ok = p >= 0 && p < max_len;
    const float inv = 1.f / powf(theta, (2.f * (float)i) / (float)HD);
    const float ang = (float)p * inv;
    const float c = l8_f(cbl_cvt_out<T>(cosf(ang))), sn = l8_f(cbl_cvt_out<T>(sinf(ang)));
    // one output element of matrix mi: take the sum, scale, round, add the bias in the 16-bit type
    auto take = [&](int mi, int r, int bcol) {
        const float y = l8_f(cbl_cvt_out<T>(__ldcg(P.fsum[mi] + r) * __half2float(((const __half*)P.m[mi].row_scale)[r])));
        return bias ? l8_f(cbl_cvt_out<T>(y + l8_f(bias[bcol]))) : y;
    };
    const bool isq = hd < NH;
    const int mi = isq ? 0 : 1, o = (isq ? hd : hd - NH) * HD, bo = hd * HD;
    const float x1 = take(mi, o + i, bo + i), x2 = take(mi, o + i + half, bo + i + half);
    const T r1 = cbl_cvt_out<T>(x1 * c - x2 * sn), r2 = cbl_cvt_out<T>(x2 * c + x1 * sn);
    if (isq) {
        if (ok) { qo[o + i] = r1; qo[o + i + half] = r2; }
    } else {
        const int kv = hd - NH, bv = (NH + NKV + kv) * HD;
        const float v1 = take(2, o + i, bv + i), v2 = take(2, o + i + half, bv + i + half);
        if (ok) {
            const int64_t co = ((int64_t)kv * max_len + p) * HD;
            kc[co + i] = r1;
            kc[co + i + half] = r2;
            const int64_t vo = (int64_t)kv * HD * max_len + p;      // values dimension-major: [kv][HD][max_len]
            vc[vo + (int64_t)i * max_len] = cbl_cvt_out<T>(v1);
            vc[vo + (int64_t)(i + half) * max_len] = cbl_cvt_out<T>(v2);
        }
    }
}

template <typename... KA, typename... A>
static int l8_finish_launch(void (*kern)(KA...), dim3 grid, dim3 block, int cluster_x, cudaStream_t st, A... args) {
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = cluster_x > 1 ? 2 : 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...));
    return cbl_check_launch();
}

extern "C" int cbl_gemv_l8_silu_mul(const cbl_l8* gate_up, const void* x, int xdtype, void* out, void* y_gate, void* y_up, int dtype,
                                    void* workspace, cbl_stream s) {
    if (!out || (dtype != CBL_F16 && dtype != CBL_BF16)) return CBL_EINVAL;
    L8Launch P;
    int rc = l8_group(gate_up, 2, x, xdtype, nullptr, dtype, 1, workspace, P);
    P.y[0] = y_gate;
    P.y[1] = y_up;
    if (rc) return rc;
    if (gate_up[0].R != gate_up[1].R) return CBL_EINVAL;
    if (P.n == 0) return CBL_OK;
    const cudaStream_t st = (cudaStream_t)s;
    rc = launch_l8(P, x, xdtype, st);
    if (rc) return rc;
    const dim3 grid(cbl_ceil_div(cbl_ceil_div(P.m[0].R, 4), 256));
    if (dtype == CBL_F16) return l8_finish_launch(k_l8_finish_silu<__half>, grid, dim3(256), 1, st, P, (__half*)out);
    return l8_finish_launch(k_l8_finish_silu<__nv_bfloat16>, grid, dim3(256), 1, st, P, (__nv_bfloat16*)out);
}

extern "C" int32_t cbl_gemv_l8_add_norm_max_rows(void) { return L8_NORM_MAX_CTAS * 1024; }

extern "C" int cbl_gemv_l8_add_norm(const cbl_l8* m, const void* x, int xdtype, float* h, const void* w, float eps, void* xout, void* y,
                                    int dtype, void* workspace, cbl_stream s) {
    if (!h || !w || !xout || (dtype != CBL_F16 && dtype != CBL_BF16)) return CBL_EINVAL;
    L8Launch P;
    int rc = l8_group(m, 1, x, xdtype, nullptr, dtype, 1, workspace, P);
    P.y[0] = y;
    if (rc) return rc;
    if (m->R < 1) return CBL_EINVAL;
    if (m->R > L8_NORM_MAX_CTAS * 1024) return CBL_EUNSUPPORTED;
    const cudaStream_t st = (cudaStream_t)s;
    rc = launch_l8(P, x, xdtype, st);
    if (rc) return rc;
    const int nb = cbl_ceil_div(cbl_ceil_div(P.m[0].R, 4), 256);
    if (dtype == CBL_F16) return l8_finish_launch(k_l8_finish_addnorm<__half>, dim3(nb), dim3(256), nb, st, P, h, (const __half*)w, eps, (__half*)xout);
    return l8_finish_launch(k_l8_finish_addnorm<__nv_bfloat16>, dim3(nb), dim3(256), nb, st, P, h, (const __nv_bfloat16*)w, eps,
                            (__nv_bfloat16*)xout);
}

extern "C" int cbl_gemv_l8_rope_kv(const cbl_l8* qkv, const void* x, int xdtype, const void* bias, const int32_t* pos, int32_t NH, int32_t NKV,
                                   int32_t HD, float theta, int32_t max_len, void* q_out, void* kc, void* vc, int dtype, void* workspace,
                                   cbl_stream s) {
    if (!pos || !q_out || !kc || !vc || (dtype != CBL_F16 && dtype != CBL_BF16) || NH < 1 || NKV < 1 || max_len < 1) return CBL_EINVAL;
    if (HD < 2 || HD > 128 || (HD & 1)) return CBL_EUNSUPPORTED;
    L8Launch P;
    int rc = l8_group(qkv, 3, x, xdtype, nullptr, dtype, 1, workspace, P);
    if (rc) return rc;
    if (qkv[0].R != NH * HD || qkv[1].R != NKV * HD || qkv[2].R != NKV * HD) return CBL_EINVAL;
    const cudaStream_t st = (cudaStream_t)s;
    rc = launch_l8(P, x, xdtype, st);
    if (rc) return rc;
    const dim3 grid(NH + NKV);
    if (dtype == CBL_F16)
        return l8_finish_launch(k_l8_finish_rope<__half>, grid, dim3(64), 1, st, P, (const __half*)bias, pos, (int)NH, (int)NKV, (int)HD, theta,
                                (int)max_len, (__half*)q_out, (__half*)kc, (__half*)vc);
    return l8_finish_launch(k_l8_finish_rope<__nv_bfloat16>, grid, dim3(64), 1, st, P, (const __nv_bfloat16*)bias, pos, (int)NH, (int)NKV, (int)HD,
                            theta, (int)max_len, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc);
}

// ------------------------------------------------------------------------------------ row-split product + sum over ranks through peer memory
//
// Tensor-parallel o / down projections: every rank multiplies its chunk range into fp32 sums in its own
// work space (the kernel above, mode 1), then ONE small kernel per rank finishes the job across GPUs without a
// collective library: it publishes "my partial sums of call e are complete" to every peer (a word
// stored into the peer's flag array over NVLink), waits - bounded - for the same word from every
// peer, reads all ranks' partial sums with plain peer loads, adds them in rank order (so every rank
// gets bit-identical results), applies the row scale and writes y.  Two sum buffers alternate
// by call so that a rank never overwrites sums a peer may still be reading.  The call number e lives
// in the work space and is advanced by the kernel itself, so a captured CUDA graph can be replayed.
//
// Work space of each rank (the same layout everywhere, allocated as symmetric memory by the caller,
// zero before the first call): sums[0] | sums[1] (rmax fp32 each) | flags (uint32 per rank) | status |
// completed calls | block ticket | the product's own partial-sum slots.
constexpr int L8_AR_MAX_RANKS = 8;
constexpr uint32_t L8_AR_SPIN_LIMIT = 1u << 22;      // polls of a peer's flag before giving up (~1 s)

struct L8AllReduce {
    int rank, world, R, ydtype;
    int64_t stride;                           // floats between the two sum buffers
    const float* sums[L8_AR_MAX_RANKS];       // every rank's sum buffer 0 (peer pointers)
    uint32_t* flags[L8_AR_MAX_RANKS];         // every rank's flag array
    uint32_t* ctl;                            // this rank's {status, completed calls, ticket}
    const __half* row_scale;
    void* y;
};

extern "C" size_t cbl_gemv_l8_ar_workspace_bytes(int32_t R) {
    if (R < 0) return 0;
    return l8_rows_max(R) * 8 + L8_AR_MAX_RANKS * 4 + 32 + L8_PART_BYTES + L8_CTL_WORDS * 4;
}

__global__ void __launch_bounds__(256) k_l8_finish_allreduce(const __grid_constant__ L8AllReduce A) {
    __shared__ int s_ok;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");          // this rank's partial sums have landed
    const int tid = threadIdx.x;
    const uint32_t epoch = __ldcg(A.ctl + 1) + 1u;              // every block reads it before the last block advances it
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < A.world) {
        // publish (one block does it), then wait for every peer's word of this call
        // (the sums were written by the kernel before this one; the release store orders them before the word)
        if (blockIdx.x == 0) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(A.flags[tid] + A.rank), "r"(epoch) : "memory");
        const uint32_t* f = A.flags[A.rank] + tid;
        bool seen = false;
        for (uint32_t i = 0; i < L8_AR_SPIN_LIMIT && !seen; i++) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            seen = (int32_t)(v - epoch) >= 0;
        }
        if (!seen) s_ok = 0;
    }
    __syncthreads();
    const int gi = blockIdx.x * blockDim.x + tid;
    if (!s_ok) {                                                // a peer never arrived: report, do not touch y
        if (tid == 0) atomicExch(A.ctl, 1u);
    } else if (gi * 4 < A.R) {
        const int64_t cur = (int64_t)(epoch & 1u) * A.stride;
        // all ranks' values are requested before the first one is used (one NVLink round trip, not one per rank),
        // then added in rank order
        float4 v[L8_AR_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < L8_AR_MAX_RANKS; r++)
            if (r < A.world) v[r] = __ldcg((const float4*)(A.sums[r] + cur) + gi);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < L8_AR_MAX_RANKS; r++)
            if (r < A.world) { sum.x += v[r].x; sum.y += v[r].y; sum.z += v[r].z; sum.w += v[r].w; }
        const float vv[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int r = gi * 4 + u;
            if (r < A.R) cbl_store_out(A.y, A.ydtype, r, vv[u] * __half2float(A.row_scale[r]));
        }
    }
    // the last block to get here advances the call counter (all blocks have read it by then)
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(A.ctl + 2, 1u) == gridDim.x - 1) {
            A.ctl[2] = 0u;
            __stcg(A.ctl + 1, epoch);
        }
    }
}

extern "C" int cbl_gemv_l8_ar(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* const* peer_ws, int32_t rank,
                              int32_t world, cbl_stream s) {
    if (!m || !x || !y || !peer_ws) return CBL_EINVAL;
    if (world < 1 || world > L8_AR_MAX_RANKS || rank < 0 || rank >= world) return CBL_EINVAL;
    int rc = check_l8r(m);
    if (rc) return rc;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    for (int r = 0; r < world; r++)
        if (!peer_ws[r] || ((uintptr_t)peer_ws[r] % 16)) return CBL_EINVAL;
    if (m->R == 0) return CBL_OK;
    const size_t rmax = l8_rows_max(m->R);
    char* own = (char*)peer_ws[rank];
    uint32_t* ctl = (uint32_t*)(own + 2 * rmax * 4 + L8_AR_MAX_RANKS * 4);
    L8Launch P;
    P.n = 1;
    P.ydtype = ydtype;
    P.mode = 1;
    P.m[0] = *m;
    P.fsum[0] = (float*)own;
    P.partial = (unsigned long long*)(own + 2 * rmax * 4 + L8_AR_MAX_RANKS * 4 + 32);
    P.y[0] = y;
    P.status = ctl;
    P.calls = ctl + 1;
    P.fsum_stride = (int64_t)rmax;
    L8AllReduce A;
    A.rank = rank; A.world = world; A.R = m->R; A.ydtype = ydtype;
    A.stride = (int64_t)rmax;
    for (int r = 0; r < world; r++) {
        A.sums[r] = (const float*)peer_ws[r];
        A.flags[r] = (uint32_t*)((char*)peer_ws[r] + 2 * rmax * 4);
    }
    A.ctl = ctl;
    A.row_scale = (const __half*)m->row_scale;
    A.y = y;
    cudaStream_t st = (cudaStream_t)s;
    rc = launch_l8(P, x, xdtype, st);
    if (rc) return rc;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(cbl_ceil_div(cbl_ceil_div(m->R, 4), 256));
    cfg.blockDim = dim3(256);
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_l8_finish_allreduce, A));
    return cbl_check_launch();
}

// Status of the last cbl_gemv_l8_ar calls on this rank's work space: CBL_ETIMEOUT if a peer's "ready" word
// did not arrive within the bounded wait (the output of that call is invalid).  Synchronises the stream
// and clears the status word.
extern "C" int cbl_gemv_l8_ar_status(void* workspace, int32_t R, cbl_stream s) {
    if (!workspace || R < 0) return CBL_EINVAL;
    char* p = (char*)workspace + 2 * l8_rows_max(R) * 4 + L8_AR_MAX_RANKS * 4;
    unsigned int v = 0;
    CBL_CUDA(cudaMemcpyAsync(&v, p, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    CBL_CUDA(cudaStreamSynchronize((cudaStream_t)s));
    if (v) CBL_CUDA(cudaMemsetAsync(p, 0, 4, (cudaStream_t)s));
    return v ? CBL_ETIMEOUT : CBL_OK;
}

// ------------------------------------------------------------------------------------ batch-1 product without caller work space
//
// Some hosts may not give this library a way to obtain device memory: a serving runtime that carves
// all of HBM into its own pools at start-up, or a plugin slot whose contract forbids allocator calls
// on the request path (an allocation can synchronise the device and fragments a pre-sized pool).
// For them the product's work space (partial-sum slots, status word) lives in a fixed array inside the
// library image instead of a caller buffer; the launch is limited to L8_STATIC_BLOCKS thread blocks so that
// the array stays small (1 MB + 256 B per GPU, part of every CUDA context that loads the library, held until
// the process exits).
constexpr int L8_STATIC_MAX_ROWS = 65536;
constexpr int L8_STATIC_BLOCKS = 32;
constexpr size_t L8_STATIC_SLOT_BYTES = (size_t)L8_STATIC_BLOCKS * L8_SLOT_ROWS * 8;
static __device__ __align__(256) unsigned char g_l8_static_scratch[L8_STATIC_SLOT_BYTES + L8_CTL_WORDS * 4];

extern "C" int32_t cbl_gemv_l8_static_max_rows(void) { return L8_STATIC_MAX_ROWS; }

// Device address of the built-in array on the current device.  The array's name is only a host-side handle; the
// address comes from the runtime, once per device, with that device current.
static int l8_static_addr(void** out) {
    static void* addr[64] = {};
    static std::mutex mu;
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CBL_EUNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        CBL_CUDA(cudaGetSymbolAddress(&p, g_l8_static_scratch));
        addr[dev] = p;
    }
    *out = addr[dev];
    return CBL_OK;
}

extern "C" int cbl_gemv_l8_static(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, cbl_stream s) {
    if (!m || !x || !y) return CBL_EINVAL;
    if (m->R > L8_STATIC_MAX_ROWS) return CBL_EUNSUPPORTED;      // stated limit of this entry point
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    void* scratch = nullptr;
    int rc = l8_static_addr(&scratch);                           // (the first call per device should happen outside stream capture)
    if (rc) return rc;
    rc = check_l8r(m);
    if (rc) return rc;
    if (m->R == 0) return CBL_OK;
    // Every call shares the array and finds whatever the previous call left.  The array starts zero (static
    // storage) and a product that ran to its end has cleared every word it used, so nothing needs clearing here;
    // a product that gave up (status word set) leaves words behind, which cbl_gemv_l8_static_status clears.
    L8Launch P;
    P.n = 1;
    P.ydtype = ydtype;
    P.mode = 0;
    P.m[0] = *m;
    P.partial = (unsigned long long*)scratch;
    P.fsum[0] = nullptr;
    P.y[0] = y;
    P.status = (unsigned int*)((char*)scratch + L8_STATIC_SLOT_BYTES) + L8_STATUS_WORD;
    P.calls = nullptr;
    P.fsum_stride = 0;
    return launch_l8(P, x, xdtype, (cudaStream_t)s, L8_STATIC_BLOCKS);
}

// CBL_ETIMEOUT if a cbl_gemv_l8_static product on the current device gave up on a bounded wait since the last
// query (its output is invalid).  Synchronises the stream; after a time-out it also clears the array on that
// stream, so the next product starts clean.  Allocates nothing.
extern "C" int cbl_gemv_l8_static_status(cbl_stream s) {
    void* scratch = nullptr;
    int rc = l8_static_addr(&scratch);
    if (rc) return rc;
    unsigned int v = 0;
    CBL_CUDA(cudaMemcpyAsync(&v, (char*)scratch + L8_STATIC_SLOT_BYTES + L8_STATUS_WORD * 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    CBL_CUDA(cudaStreamSynchronize((cudaStream_t)s));
    if (v) CBL_CUDA(cudaMemsetAsync(scratch, 0, L8_STATIC_SLOT_BYTES + L8_CTL_WORDS * 4, (cudaStream_t)s));
    return v ? CBL_ETIMEOUT : CBL_OK;
}
