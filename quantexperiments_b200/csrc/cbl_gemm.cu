// Prefill product Y[tokens, R] = X[tokens, C] . W^T with W decoded on the fly into shared memory and
// multiplied on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// One thread block computes a 256-token x 256-row tile: two 128 x 256 fp32 accumulators fill the 512
// TMEM columns.  Per 64-wide k-block
//   - one thread brings the activations (fp16, two 128 x 64 boxes) in with TMA, 128-byte swizzled;
//   - 256 decode threads, one per W row, read the row's eight 12-bit tags, fetch the eight 16-byte
//     codewords from the 64 KB book in shared memory and store them into the K-major 128-byte
//     swizzled B tile (one codeword = one 16-byte swizzle unit), then fence to the async proxy;
//   - one thread issues 2 x 4 tcgen05.mma (M 128, N 256, K 16, fp16 x fp16 -> fp32) and commits to
//     the stage's "empty" barrier.
// The epilogue reads TMEM with tcgen05.ld, applies the fp16 row scale and the token's power-of-two
// activation scale, rounds once and writes Y.  Every wait is bounded; a wait that expires sets the
// status word and lets the block drain and free its tensor memory.
#include <cuda.h>
#include "cbl_common.cuh"

namespace {

constexpr int GM_BM = 256;                 // tokens per tile (2 accumulators of 128)
constexpr int GM_BN = 256;                 // W rows per tile (UMMA N)
constexpr int GM_BK = 64;                  // k-block: 8 chunks, one 128-byte swizzled row
constexpr int GM_A_STAGES = 3;             // activation (TMA) ring: 3 x 32 KB
constexpr int GM_B_STAGES = 2;             // decoded weight ring: 2 x 32 KB
constexpr int GM_A_BYTES = 128 * GM_BK * 2;            // one 128-token box
constexpr int GM_B_BYTES = GM_BN * GM_BK * 2;
constexpr int GM_SMEM = 65536 + GM_A_STAGES * 2 * GM_A_BYTES + GM_B_STAGES * GM_B_BYTES;   // book + rings = 224 KB
constexpr int GM_DECODE_WARPS = 8, GM_THREADS = (GM_DECODE_WARPS + 2) * 32;
constexpr uint32_t GM_WAIT_LIMIT = 1u << 24;   // mbarrier polls (a few tens of cycles each) before a wait gives up

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for a phase of an mbarrier: a non-blocking test in a spin loop (the blocking try_wait form
// adds wake-up latency to every pipeline hand-off); false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < GM_WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart (descriptor version 1).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

// One token's 32 consecutive outputs: row scales as four 16-byte loads, outputs as 16-byte stores when aligned.
__device__ __forceinline__ void gemm_store_row32(const uint32_t (&v)[32], int tok, int ntok, int rbase, const cbl_l8& m, float tsc,
                                                 void* __restrict__ y, int ydtype, int64_t ldy, int vec_ok) {
    if (tok >= ntok || rbase >= m.R) return;
    if (vec_ok && rbase + 32 <= m.R) {
        union { uint4 u[4]; __half h[32]; } rsv;
        const uint4* rp = (const uint4*)((const __half*)m.row_scale + rbase);
#pragma unroll
        for (int j = 0; j < 4; j++) rsv.u[j] = __ldg(rp + j);
        float o[32];
#pragma unroll
        for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]) * tsc * __half2float(rsv.h[j]);
        if (ydtype == CBL_F32) {
            float4* dst = (float4*)((float*)y + (int64_t)tok * ldy + rbase);
#pragma unroll
            for (int j = 0; j < 8; j++) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        } else {
            union { uint4 u[4]; __nv_bfloat16 b[32]; __half h[32]; } pk;
            if (ydtype == CBL_BF16) {
#pragma unroll
                for (int j = 0; j < 32; j++) pk.b[j] = __float2bfloat16_rn(o[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) pk.h[j] = __float2half_rn(o[j]);
            }
            uint4* dst = (uint4*)((char*)y + ((int64_t)tok * ldy + rbase) * 2);
#pragma unroll
            for (int j = 0; j < 4; j++) dst[j] = pk.u[j];
        }
    } else {
#pragma unroll 1
        for (int j = 0; j < 32; j++) {
            const int r = rbase + j;
            if (r < m.R) {
                const float rs = __half2float(__ldg((const __half*)m.row_scale + r));
                cbl_store_out(y, ydtype, (int64_t)tok * ldy + r, __uint_as_float(v[j]) * tsc * rs);
            }
        }
    }
}

__global__ void __launch_bounds__(GM_THREADS, 1)
k_gemm_l8(const __grid_constant__ CUtensorMap xmap, cbl_l8 m, const float* __restrict__ xinv, int ntok, void* __restrict__ y, int ydtype,
          int64_t ldy, int vec_ok, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // barriers: full_a / empty_a per activation stage, full_b / empty_b per weight stage, tmem_full
    __shared__ __align__(8) unsigned long long s_bar[2 * GM_A_STAGES + 2 * GM_B_STAGES + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // row tiles vary fastest across the grid: blocks that run together share one activation tile in L2
    const int r0 = blockIdx.x * GM_BN, tok0 = blockIdx.y * GM_BM;
    // one tile of the l8 layout per k-block; a second (summed) book is a second pass over the same activation
    // k-blocks with the other book in shared memory: Y = X A^T + X B^T accumulates in the same tensor memory
    const int nkb = m.ntile, nkb1 = m.ntile / m.books;
    const uint32_t sbase = cbl_smem_u32(smem), bar0 = cbl_smem_u32(s_bar);
    auto full_a = [&](int s) { return bar0 + 8u * s; };
    auto empty_a = [&](int s) { return bar0 + 8u * (GM_A_STAGES + s); };
    auto full_b = [&](int s) { return bar0 + 8u * (2 * GM_A_STAGES + s); };
    auto empty_b = [&](int s) { return bar0 + 8u * (2 * GM_A_STAGES + GM_B_STAGES + s); };
    const uint32_t tmem_full = bar0 + 8u * (2 * GM_A_STAGES + 2 * GM_B_STAGES);
    const uint32_t a_base = sbase + 65536, b_base = a_base + GM_A_STAGES * 2 * GM_A_BYTES;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < GM_A_STAGES; s++) { mbar_init(full_a(s), 1); mbar_init(empty_a(s), 1); }
        for (int s = 0; s < GM_B_STAGES; s++) { mbar_init(full_b(s), GM_DECODE_WARPS); mbar_init(empty_b(s), 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == GM_DECODE_WARPS) {                            // this warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the book: 4096 codewords of 16 bytes
    if (warp < GM_DECODE_WARPS) {
        const uint4* t0 = (const uint4*)m.table;
        uint4* dst = (uint4*)smem;
        for (int i = tid; i < 4096; i += GM_DECODE_WARPS * 32) dst[i] = __ldg(t0 + i);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == GM_DECODE_WARPS) {
        // ---------------- TMA producer of the activations (its ring is deeper than the weights': the
        // round trip through L2 is several k-blocks long)
        if (lane == 0) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % GM_A_STAGES;
                if (!mbar_wait(empty_a(s), ((kb / GM_A_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
                mbar_expect_tx(full_a(s), 2 * GM_A_BYTES);
                const uint32_t dst = a_base + s * 2 * GM_A_BYTES;
                const int kx = (kb >= nkb1 ? kb - nkb1 : kb) * GM_BK;
                tma_load_2d(dst, &xmap, kx, tok0, full_a(s));
                tma_load_2d(dst + GM_A_BYTES, &xmap, kx, tok0 + 128, full_a(s));
            }
        }
    } else if (warp == GM_DECODE_WARPS + 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(GM_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f16 x f16 -> f32, K-major both
            for (int kb = 0; kb < nkb; kb++) {
                const int sa = kb % GM_A_STAGES, sb = kb % GM_B_STAGES;
                if (!(mbar_wait(full_a(sa), (kb / GM_A_STAGES) & 1) && mbar_wait(full_b(sb), (kb / GM_B_STAGES) & 1))) { s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = a_base + sa * 2 * GM_A_BYTES, b_addr = b_base + sb * GM_B_BYTES;
#pragma unroll
                for (int tb = 0; tb < 2; tb++) {
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; kk++) {
                        const uint64_t da = umma_desc_sw128(a_addr + tb * GM_A_BYTES + kk * 32);
                        const uint64_t db = umma_desc_sw128(b_addr + kk * 32);
                        umma_f16(tmem + tb * GM_BN, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                }
                umma_commit(empty_a(sa));
                umma_commit(empty_b(sb));
            }
            umma_commit(tmem_full);       // arrives when every MMA issued so far has completed
        }
    } else {
        // ---------------- decode: thread t owns W row r0 + t of the tile
        const int row = r0 + tid;
        const bool live = row < m.Rpad;
        const uint32_t* wp = (const uint32_t*)m.words + row;
        // this row's tag words of the current and the next two k-blocks (three words each)
        uint32_t wa = 0, wb = 0, wc = 0, na = 0, nb = 0, nc = 0, fa = 0, fb = 0, fc = 0;
        auto load_tags = [&](int kb, uint32_t& a, uint32_t& b, uint32_t& c) {
            a = b = c = 0;
            if (live && kb < nkb) {
                const uint32_t* p = wp + (int64_t)kb * 3 * m.Rpad;
                a = __ldg(p); b = __ldg(p + m.Rpad); c = __ldg(p + 2 * (int64_t)m.Rpad);
            }
        };
        load_tags(0, wa, wb, wc);
        load_tags(1, na, nb, nc);
        const uint32_t sw = (uint32_t)(tid & 7);
        const uint32_t rowoff = (uint32_t)(tid >> 3) * 1024u + sw * 128u;
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % GM_B_STAGES;
            load_tags(kb + 2, fa, fb, fc);
            if (kb == nkb1 && m.books == 2) {
                // switch books: every decode thread is done with the first one (barrier among the decode warps only)
                asm volatile("bar.sync 1, %0;" ::"n"(GM_DECODE_WARPS * 32) : "memory");
                const uint4* t1 = (const uint4*)m.table2;
                uint4* dst = (uint4*)smem;
                for (int i = tid; i < 4096; i += GM_DECODE_WARPS * 32) dst[i] = __ldg(t1 + i);
                asm volatile("bar.sync 1, %0;" ::"n"(GM_DECODE_WARPS * 32) : "memory");
            }
            if (!mbar_wait(empty_b(s), ((kb / GM_B_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
            const uint32_t bdst = b_base + s * GM_B_BYTES + rowoff;
            uint32_t off[8];
            off[0] = (wa << 4) & 0xFFF0u;
            off[1] = (wa >> 8) & 0xFFF0u;
            off[2] = __funnelshift_r(wa, wb, 20) & 0xFFF0u;
            off[3] = wb & 0xFFF0u;
            off[4] = (wb >> 12) & 0xFFF0u;
            off[5] = __funnelshift_r(wb, wc, 24) & 0xFFF0u;
            off[6] = (wc >> 4) & 0xFFF0u;
            off[7] = (wc >> 16) & 0xFFF0u;
            uint4 cw[8];
#pragma unroll
            for (int c = 0; c < 8; c++) cw[c] = cbl_lds128(sbase + off[c]);      // all eight gathers in flight before the stores
#pragma unroll
            for (int c = 0; c < 8; c++)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bdst + (((uint32_t)c ^ sw) << 4)), "r"(cw[c].x), "r"(cw[c].y),
                             "r"(cw[c].z), "r"(cw[c].w)
                             : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full_b(s));
            wa = na; wb = nb; wc = nc;
            na = fa; nb = fb; nc = fc;
        }
        // ---------------- epilogue: warp w reads TMEM lanes 32*(w%4).. of accumulator w/4
        const bool ok = mbar_wait(tmem_full, 0);
        if (!ok) s_abort = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3, tb = warp >> 2;
        const int tok = tok0 + tb * 128 + q * 32 + lane;
        const float tsc = (tok < ntok) ? xinv[tok] : 0.f;
        if (ok) {
            for (int c0 = 0; c0 < GM_BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(tb * GM_BN + c0), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                gemm_store_row32(v, tok, ntok, r0 + c0, m, tsc, y, ydtype, ldy, vec_ok);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    if (warp == GM_DECODE_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------ two-SM variant
//
// A cluster of two blocks computes a 512-token x 256-row tile with tcgen05.mma.cta_group::2 (M 256 split
// over the two SMs, N 256).  Each block loads its own 2 x 128 tokens of activations and decodes only
// HALF of the B tile (128 W rows), so the shared-memory cost of decoding per MMA cycle halves.  The MMA
// is issued by the leader block (cluster rank 0); "full" barriers live in the leader and are signalled by
// both blocks (TMA complete_tx and remote arrives), "empty" and "accumulators ready" are multicast
// commits to both blocks.
constexpr int G2_STAGES = 3;
constexpr int G2_B_BYTES = 128 * GM_BK * 2;                              // this block's half of the B tile
constexpr int G2_STAGE_BYTES = 2 * GM_A_BYTES + G2_B_BYTES;              // 48 KB
constexpr int G2_SMEM = 65536 + G2_STAGES * G2_STAGE_BYTES;
constexpr int G2_DECODE_WARPS = 4, G2_THREADS = (G2_DECODE_WARPS + 2) * 32;

__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_2sm(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
                 : "memory");
}
__device__ __forceinline__ void umma_f16_2sm(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(G2_THREADS, 1)
k_gemm_l8_2sm(const __grid_constant__ CUtensorMap xmap, cbl_l8 m, const float* __restrict__ xinv, int ntok, void* __restrict__ y, int ydtype,
              int64_t ldy, int vec_ok, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[3 * G2_STAGES + 1];   // full_a, full_b, empty per stage; tmem_full
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int r0 = (blockIdx.x >> 1) * GM_BN, tok_base = blockIdx.y * 512;
    const int nkb = m.ntile;
    const uint32_t sbase = cbl_smem_u32(smem), bar0 = cbl_smem_u32(s_bar);
    auto full_a = [&](int s) { return bar0 + 8u * s; };
    auto full_b = [&](int s) { return bar0 + 8u * (G2_STAGES + s); };
    auto empty = [&](int s) { return bar0 + 8u * (2 * G2_STAGES + s); };
    const uint32_t tmem_full = bar0 + 8u * (3 * G2_STAGES);

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < G2_STAGES; s++) {
            mbar_init(full_a(s), 1);                          // the leader's expect_tx arrival; bytes come from both blocks
            mbar_init(full_b(s), 2 * G2_DECODE_WARPS);        // decode warps of both blocks
            mbar_init(empty(s), 1);
        }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == G2_DECODE_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    if (warp < G2_DECODE_WARPS) {
        const uint4* t0 = (const uint4*)m.table;
        uint4* dst = (uint4*)smem;
        for (int i = tid; i < 4096; i += G2_DECODE_WARPS * 32) dst[i] = __ldg(t0 + i);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                        // both blocks' barriers and tensor memory exist
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == G2_DECODE_WARPS) {
        // ---------------- TMA producer: this block's 2 x 128 tokens; completion lands on the leader's barrier
        if (lane == 0) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % G2_STAGES;
                if (!mbar_wait(empty(s), ((kb / G2_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
                if (rank == 0) mbar_expect_tx(full_a(s), 2 * 2 * GM_A_BYTES);
                const uint32_t dst = sbase + 65536 + s * G2_STAGE_BYTES;
                const uint32_t lead_bar = mapa_u32(full_a(s), 0);
                tma_load_2d_2sm(dst, &xmap, kb * GM_BK, tok_base + (int)rank * 128, lead_bar);
                tma_load_2d_2sm(dst + GM_A_BYTES, &xmap, kb * GM_BK, tok_base + 256 + (int)rank * 128, lead_bar);
            }
        }
    } else if (warp == G2_DECODE_WARPS + 1) {
        // ---------------- MMA issuer (leader block only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(GM_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % G2_STAGES;
                const uint32_t par = (kb / G2_STAGES) & 1;
                if (!(mbar_wait(full_a(s), par) && mbar_wait(full_b(s), par))) { s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = sbase + 65536 + s * G2_STAGE_BYTES, b_addr = a_addr + 2 * GM_A_BYTES;
#pragma unroll
                for (int tb = 0; tb < 2; tb++) {
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; kk++) {
                        const uint64_t da = umma_desc_sw128(a_addr + tb * GM_A_BYTES + kk * 32);
                        const uint64_t db = umma_desc_sw128(b_addr + kk * 32);
                        umma_f16_2sm(tmem + tb * GM_BN, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                }
                umma_commit_2sm(empty(s));
            }
            umma_commit_2sm(tmem_full);
        }
    } else {
        // ---------------- decode: thread t owns W row r0 + 128*rank + t (this block's half of the B tile)
        const int row = r0 + (int)rank * 128 + tid;
        const bool live = row < m.Rpad;
        const uint32_t* wp = (const uint32_t*)m.words + row;
        uint32_t wa = 0, wb = 0, wc = 0, na = 0, nb = 0, nc = 0, fa = 0, fb = 0, fc = 0;
        auto load_tags = [&](int kb, uint32_t& a, uint32_t& b, uint32_t& c) {
            a = b = c = 0;
            if (live && kb < nkb) {
                const uint32_t* p = wp + (int64_t)kb * 3 * m.Rpad;
                a = __ldg(p); b = __ldg(p + m.Rpad); c = __ldg(p + 2 * (int64_t)m.Rpad);
            }
        };
        load_tags(0, wa, wb, wc);
        load_tags(1, na, nb, nc);
        const uint32_t sw = (uint32_t)(tid & 7);
        const uint32_t rowoff = (uint32_t)(tid >> 3) * 1024u + sw * 128u;
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % G2_STAGES;
            load_tags(kb + 2, fa, fb, fc);
            if (!mbar_wait(empty(s), ((kb / G2_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
            const uint32_t bdst = sbase + 65536 + s * G2_STAGE_BYTES + 2 * GM_A_BYTES + rowoff;
            uint32_t off[8];
            off[0] = (wa << 4) & 0xFFF0u;
            off[1] = (wa >> 8) & 0xFFF0u;
            off[2] = __funnelshift_r(wa, wb, 20) & 0xFFF0u;
            off[3] = wb & 0xFFF0u;
            off[4] = (wb >> 12) & 0xFFF0u;
            off[5] = __funnelshift_r(wb, wc, 24) & 0xFFF0u;
            off[6] = (wc >> 4) & 0xFFF0u;
            off[7] = (wc >> 16) & 0xFFF0u;
            uint4 cw[8];
#pragma unroll
            for (int c = 0; c < 8; c++) cw[c] = cbl_lds128(sbase + off[c]);      // all eight gathers in flight before the stores
#pragma unroll
            for (int c = 0; c < 8; c++)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(bdst + (((uint32_t)c ^ sw) << 4)), "r"(cw[c].x), "r"(cw[c].y),
                             "r"(cw[c].z), "r"(cw[c].w)
                             : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(full_b(s), 0));
            wa = na; wb = nb; wc = nc;
            na = fa; nb = fb; nc = fc;
        }
        // ---------------- epilogue: warp q reads TMEM lanes 32q.. of both accumulators of this block
        const bool ok = mbar_wait(tmem_full, 0);
        if (!ok) s_abort = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3;
        if (ok) {
            for (int tb = 0; tb < 2; tb++) {
                const int tok = tok_base + tb * 256 + (int)rank * 128 + q * 32 + lane;
                const float tsc = (tok < ntok) ? xinv[tok] : 0.f;
                for (int c0 = 0; c0 < GM_BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(tb * GM_BN + c0), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    gemm_store_row32(v, tok, ntok, r0 + c0, m, tsc, y, ydtype, ldy, vec_ok);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    cluster_sync_all();                                        // the peer no longer reads or signals this block's memory
    if (warp == G2_DECODE_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------ up to 32 tokens: weight rows as M
//
// For a handful of tokens the product is bound by decoding alone, so the tile is turned around: 128 weight rows
// are the M side of tcgen05.mma (decoded into the K-major swizzled A tile), the tokens the N side (16 or 32,
// brought in by TMA).  Every weight is decoded exactly once whatever the token count, the MMAs are negligible,
// and there are no per-step activation fragments to fetch as in the mma.sync kernel.  512 decode threads = 128
// rows x 4 k-blocks per hand-off (64 KB of A per stage, two stages).  Blocks = (row tile, k part): products with
// few row tiles are split along k and summed with fp32 reductions into a work space, finished by a second
// kernel.  Up to four matrices that share the activations run as one launch (each block stages its own
// matrix's book).
constexpr int GR_ROWS = 128;
constexpr int GR_KBS = 4;                                  // k-blocks per stage
constexpr int GR_STAGES = 2;
constexpr int GR_NMAX = 32;                                // tokens per launch
constexpr int GR_A_KB = GR_ROWS * 128;                     // one k-block of A: 16 KB
constexpr int GR_X_KB = GR_NMAX * 128;                     // one k-block of the activations: 4 KB
constexpr int GR_A_STAGE = GR_KBS * GR_A_KB, GR_X_STAGE = GR_KBS * GR_X_KB;
constexpr int GR_SMEM = 65536 + GR_STAGES * (GR_A_STAGE + GR_X_STAGE);   // 224 KB
constexpr int GR_DECODE_WARPS = 16, GR_THREADS = (GR_DECODE_WARPS + 2) * 32;
constexpr int GR_MAX_GROUP = 4;

struct GRLaunch {
    int n;                            // matrices
    int tile0[GR_MAX_GROUP + 1];      // prefix sums of their row-tile counts
    cbl_l8 m[GR_MAX_GROUP];
    float* acc[GR_MAX_GROUP];         // fp32 [npad][Rpad] partial sums (k-split launches)
    void* y[GR_MAX_GROUP];
    int ksplit, npad;
};

__global__ void __launch_bounds__(GR_THREADS, 1)
k_gemm_rows(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ GRLaunch P, const float* __restrict__ xinv, int ntok, int ydtype,
            int64_t ldy, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[3 * GR_STAGES + 1];    // full_a, full_x, empty per stage; tmem_full
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int mi = 0;
    while (mi + 1 < P.n && (int)blockIdx.x >= P.tile0[mi + 1]) mi++;
    const cbl_l8& m = P.m[mi];
    const int r0 = ((int)blockIdx.x - P.tile0[mi]) * GR_ROWS;
    const int nkb = m.ntile, nkb1 = m.ntile / m.books;
    // this block's k-blocks: part blockIdx.y of ksplit equal parts
    const int kb_lo = (int)(((int64_t)nkb * blockIdx.y) / P.ksplit), kb_hi = (int)(((int64_t)nkb * (blockIdx.y + 1)) / P.ksplit);
    const uint32_t sbase = cbl_smem_u32(smem), bar0 = cbl_smem_u32(s_bar);
    auto full_a = [&](int s) { return bar0 + 8u * s; };
    auto full_x = [&](int s) { return bar0 + 8u * (GR_STAGES + s); };
    auto empty = [&](int s) { return bar0 + 8u * (2 * GR_STAGES + s); };
    const uint32_t tmem_full = bar0 + 8u * (3 * GR_STAGES);
    const uint32_t a_base = sbase + 65536, x_base = a_base + GR_STAGES * GR_A_STAGE;
    // stages never straddle the two books: segment 0 = this part's k-blocks of the first book, segment 1 = of the second
    const int seg_lo[2] = {kb_lo < nkb1 ? kb_lo : nkb1, kb_lo > nkb1 ? kb_lo : nkb1};
    const int seg_hi[2] = {kb_hi < nkb1 ? kb_hi : nkb1, kb_hi > nkb1 ? kb_hi : nkb1};

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < GR_STAGES; s++) { mbar_init(full_a(s), GR_DECODE_WARPS); mbar_init(full_x(s), 1); mbar_init(empty(s), 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == GR_DECODE_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(32u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < GR_DECODE_WARPS) {                              // the book of the first segment that has work
        const uint4* t0 = (const uint4*)((seg_lo[0] < seg_hi[0]) ? m.table : m.table2);
        uint4* dst = (uint4*)smem;
        for (int i = tid; i < 4096; i += GR_DECODE_WARPS * 32) dst[i] = __ldg(t0 + i);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    asm volatile("griddepcontrol.wait;" ::: "memory");          // the staged activations (and zeroed sums) come from earlier kernels
    // A wait that expires marks the block aborted; every thread then keeps the shape of its loops (the decode
    // warps meet at a named barrier when the book changes) but waits for nothing more.
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (*(volatile int*)&s_abort) return;
        if (!mbar_wait(bar, parity)) s_abort = 1;
    };

    if (warp == GR_DECODE_WARPS) {
        if (lane == 0) {                                      // TMA producer of the activations
            int it = 0;
            for (int sg = 0; sg < 2; sg++) {
                for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                    const int s = it % GR_STAGES, nv = min(GR_KBS, seg_hi[sg] - kb);
                    wait(empty(s), ((it / GR_STAGES) & 1) ^ 1);
                    if (*(volatile int*)&s_abort) break;              // no copies after an abort: nothing would wait for them
                    mbar_expect_tx(full_x(s), (uint32_t)nv * (uint32_t)P.npad * 128u);
                    for (int j = 0; j < nv; j++)
                        tma_load_2d(x_base + s * GR_X_STAGE + j * GR_X_KB, &xmap, (kb + j - sg * nkb1) * GM_BK, 0, full_x(s));
                }
            }
        }
    } else if (warp == GR_DECODE_WARPS + 1) {
        if (lane == 0) {                                      // MMA issuer
            const uint32_t idesc = (1u << 4) | ((uint32_t)(P.npad >> 3) << 17) | ((uint32_t)(GR_ROWS >> 4) << 24);
            int it = 0;
            uint32_t accumulate = 0;
            for (int sg = 0; sg < 2; sg++) {
                for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                    const int s = it % GR_STAGES, nv = min(GR_KBS, seg_hi[sg] - kb);
                    const uint32_t par = (it / GR_STAGES) & 1;
                    wait(full_x(s), par);
                    wait(full_a(s), par);
                    if (*(volatile int*)&s_abort) break;              // no MMAs on tiles that never arrived
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int j = 0; j < nv; j++) {
#pragma unroll
                        for (int kk = 0; kk < GM_BK / 16; kk++) {
                            umma_f16(tmem, umma_desc_sw128(a_base + s * GR_A_STAGE + j * GR_A_KB + kk * 32),
                                     umma_desc_sw128(x_base + s * GR_X_STAGE + j * GR_X_KB + kk * 32), idesc, accumulate);
                            accumulate = 1;
                        }
                    }
                    umma_commit(empty(s));
                }
            }
            umma_commit(tmem_full);
        }
    } else {
        // ---------------- decode: thread = (W row r0 + (tid & 127), k-block tid >> 7 of the stage)
        const int rl = tid & 127, kbs = tid >> 7, row = r0 + rl;
        const bool live = row < m.Rpad;
        const uint32_t* wp = (const uint32_t*)m.words + row;
        const uint32_t sw = (uint32_t)(rl & 7);
        const uint32_t rowoff = (uint32_t)kbs * GR_A_KB + (uint32_t)(rl >> 3) * 1024u + sw * 128u;
        int it = 0;
        for (int sg = 0; sg < 2; sg++) {
            if (seg_lo[sg] >= seg_hi[sg]) continue;
            if (sg == 1 && seg_lo[0] < seg_hi[0]) {
                // switch books: every decode thread is done with the first one (barrier among the decode warps only)
                asm volatile("bar.sync 1, %0;" ::"n"(GR_DECODE_WARPS * 32) : "memory");
                const uint4* t1 = (const uint4*)m.table2;
                uint4* dst = (uint4*)smem;
                for (int i = tid; i < 4096; i += GR_DECODE_WARPS * 32) dst[i] = __ldg(t1 + i);
                asm volatile("bar.sync 1, %0;" ::"n"(GR_DECODE_WARPS * 32) : "memory");
            }
            uint32_t wa = 0, wb = 0, wc = 0, na = 0, nb = 0, nc = 0;
            auto load_tags = [&](int kb, uint32_t& a, uint32_t& b, uint32_t& c) {
                a = b = c = 0;
                if (live && kb < seg_hi[sg]) {
                    const uint32_t* p = wp + (int64_t)kb * 3 * m.Rpad;
                    a = __ldg(p); b = __ldg(p + m.Rpad); c = __ldg(p + 2 * (int64_t)m.Rpad);
                }
            };
            load_tags(seg_lo[sg] + kbs, wa, wb, wc);
            for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                const int s = it % GR_STAGES;
                load_tags(kb + GR_KBS + kbs, na, nb, nc);
                wait(empty(s), ((it / GR_STAGES) & 1) ^ 1);
                if (kb + kbs < seg_hi[sg]) {
                    const uint32_t dst = a_base + s * GR_A_STAGE + rowoff;
                    uint32_t off[8];
                    off[0] = (wa << 4) & 0xFFF0u;
                    off[1] = (wa >> 8) & 0xFFF0u;
                    off[2] = __funnelshift_r(wa, wb, 20) & 0xFFF0u;
                    off[3] = wb & 0xFFF0u;
                    off[4] = (wb >> 12) & 0xFFF0u;
                    off[5] = __funnelshift_r(wb, wc, 24) & 0xFFF0u;
                    off[6] = (wc >> 4) & 0xFFF0u;
                    off[7] = (wc >> 16) & 0xFFF0u;
                    uint4 cw[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) cw[c] = cbl_lds128(sbase + off[c]);
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (((uint32_t)c ^ sw) << 4)), "r"(cw[c].x), "r"(cw[c].y),
                                     "r"(cw[c].z), "r"(cw[c].w)
                                     : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(s));
                wa = na; wb = nb; wc = nc;
            }
        }
        // ---------------- epilogue: decode warps 0..3 read TMEM lanes (= W rows) 32 w ..; columns = tokens
        if (warp < 4) {
            wait(tmem_full, 0);
            const bool ok = *(volatile int*)&s_abort == 0;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = r0 + warp * 32 + lane;
            if (ok) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < m.R) {
                    if (P.ksplit == 1) {
                        const float rs = __half2float(__ldg((const __half*)m.row_scale + r));
#pragma unroll 4
                        for (int n = 0; n < GR_NMAX; n++)
                            if (n < ntok) cbl_store_out(P.y[mi], ydtype, (int64_t)n * ldy + r, __uint_as_float(v[n]) * xinv[n] * rs);
                    } else {
                        float* acc = P.acc[mi] + r;
#pragma unroll 4
                        for (int n = 0; n < GR_NMAX; n++)
                            if (n < ntok) atomicAdd(acc + (int64_t)n * m.Rpad, __uint_as_float(v[n]));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    if (warp == GR_DECODE_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32u) : "memory");
    }
}

// Variant with the decoded A tile in TENSOR memory: a decode thread writes its row's codewords straight from
// registers into its TMEM lane (tcgen05.st) and the MMA takes A from TMEM, so neither the store of the A tile nor
// the tensor cores' read of it touch shared memory - only the codeword gathers do.  TMEM columns: 0..31 the
// accumulator, then GT_STAGES stages of 4 k-blocks x 32 columns (a k-block = 64 fp16 per row = 32 columns).
// What bounds it now is the tensor pipe itself: an MMA of 128 rows x 16 k takes about 170 cycles however few the
// tokens (independent accumulators and a software-pipelined decode loop changed nothing), i.e. 1.4 us per stage.
constexpr int GT_STAGES = 3;
constexpr int GT_A_COL0 = 32, GT_A_STAGE_COLS = GR_KBS * 32;
constexpr int GT_SMEM = 65536 + GT_STAGES * GR_X_STAGE;

__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint4 (&c)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(c[0].x), "r"(c[0].y), "r"(c[0].z), "r"(c[0].w), "r"(c[1].x), "r"(c[1].y), "r"(c[1].z), "r"(c[1].w), "r"(c[2].x),
          "r"(c[2].y), "r"(c[2].z), "r"(c[2].w), "r"(c[3].x), "r"(c[3].y), "r"(c[3].z), "r"(c[3].w), "r"(c[4].x), "r"(c[4].y), "r"(c[4].z),
          "r"(c[4].w), "r"(c[5].x), "r"(c[5].y), "r"(c[5].z), "r"(c[5].w), "r"(c[6].x), "r"(c[6].y), "r"(c[6].z), "r"(c[6].w), "r"(c[7].x),
          "r"(c[7].y), "r"(c[7].z), "r"(c[7].w)
        : "memory");
}

__global__ void __launch_bounds__(GR_THREADS, 1)
k_gemm_rows_ta(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ GRLaunch P, const float* __restrict__ xinv, int ntok, int ydtype,
            int64_t ldy, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bar[3 * GT_STAGES + 1];    // full_a, full_x, empty per stage; tmem_full
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int mi = 0;
    while (mi + 1 < P.n && (int)blockIdx.x >= P.tile0[mi + 1]) mi++;
    const cbl_l8& m = P.m[mi];
    const int r0 = ((int)blockIdx.x - P.tile0[mi]) * GR_ROWS;
    const int nkb = m.ntile, nkb1 = m.ntile / m.books;
    // this block's k-blocks: part blockIdx.y of ksplit equal parts
    const int kb_lo = (int)(((int64_t)nkb * blockIdx.y) / P.ksplit), kb_hi = (int)(((int64_t)nkb * (blockIdx.y + 1)) / P.ksplit);
    const uint32_t sbase = cbl_smem_u32(smem), bar0 = cbl_smem_u32(s_bar);
    auto full_a = [&](int s) { return bar0 + 8u * s; };
    auto full_x = [&](int s) { return bar0 + 8u * (GT_STAGES + s); };
    auto empty = [&](int s) { return bar0 + 8u * (2 * GT_STAGES + s); };
    const uint32_t tmem_full = bar0 + 8u * (3 * GT_STAGES);
    const uint32_t x_base = sbase + 65536;
    // stages never straddle the two books: segment 0 = this part's k-blocks of the first book, segment 1 = of the second
    const int seg_lo[2] = {kb_lo < nkb1 ? kb_lo : nkb1, kb_lo > nkb1 ? kb_lo : nkb1};
    const int seg_hi[2] = {kb_hi < nkb1 ? kb_hi : nkb1, kb_hi > nkb1 ? kb_hi : nkb1};

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < GT_STAGES; s++) { mbar_init(full_a(s), GR_DECODE_WARPS); mbar_init(full_x(s), 1); mbar_init(empty(s), 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == GR_DECODE_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < GR_DECODE_WARPS) {                              // the book of the first segment that has work
        const uint4* t0 = (const uint4*)((seg_lo[0] < seg_hi[0]) ? m.table : m.table2);
        uint4* dst = (uint4*)smem;
        for (int i = tid; i < 4096; i += GR_DECODE_WARPS * 32) dst[i] = __ldg(t0 + i);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // A wait that expires marks the block aborted; every thread then keeps the shape of its loops (the decode
    // warps meet at a named barrier when the book changes) but waits for nothing more.
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (*(volatile int*)&s_abort) return;
        if (!mbar_wait(bar, parity)) s_abort = 1;
    };

    if (warp == GR_DECODE_WARPS) {
        if (lane == 0) {                                      // TMA producer of the activations
            int it = 0;
            for (int sg = 0; sg < 2; sg++) {
                for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                    const int s = it % GT_STAGES, nv = min(GR_KBS, seg_hi[sg] - kb);
                    wait(empty(s), ((it / GT_STAGES) & 1) ^ 1);
                    if (*(volatile int*)&s_abort) break;              // no copies after an abort: nothing would wait for them
                    mbar_expect_tx(full_x(s), (uint32_t)nv * (uint32_t)P.npad * 128u);
                    for (int j = 0; j < nv; j++)
                        tma_load_2d(x_base + s * GR_X_STAGE + j * GR_X_KB, &xmap, (kb + j - sg * nkb1) * GM_BK, 0, full_x(s));
                }
            }
        }
    } else if (warp == GR_DECODE_WARPS + 1) {
        if (lane == 0) {                                      // MMA issuer
            const uint32_t idesc = (1u << 4) | ((uint32_t)(P.npad >> 3) << 17) | ((uint32_t)(GR_ROWS >> 4) << 24);
            int it = 0;
            uint32_t accumulate = 0;
            for (int sg = 0; sg < 2; sg++) {
                for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                    const int s = it % GT_STAGES, nv = min(GR_KBS, seg_hi[sg] - kb);
                    const uint32_t par = (it / GT_STAGES) & 1;
                    wait(full_x(s), par);
                    wait(full_a(s), par);
                    if (*(volatile int*)&s_abort) break;              // no MMAs on tiles that never arrived
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int j = 0; j < nv; j++) {
#pragma unroll
                        for (int kk = 0; kk < GM_BK / 16; kk++) {
                            umma_f16_ta(tmem, tmem + GT_A_COL0 + s * GT_A_STAGE_COLS + j * 32 + kk * 8,
                                        umma_desc_sw128(x_base + s * GR_X_STAGE + j * GR_X_KB + kk * 32), idesc, accumulate);
                            accumulate = 1;
                        }
                    }
                    umma_commit(empty(s));
                }
            }
            umma_commit(tmem_full);
        }
    } else {
        // ---------------- decode: thread = (W row r0 + (tid & 127), k-block tid >> 7 of the stage)
        const int rl = tid & 127, kbs = tid >> 7, row = r0 + rl;
        const bool live = row < m.Rpad;
        const uint32_t* wp = (const uint32_t*)m.words + row;
        int it = 0;
        for (int sg = 0; sg < 2; sg++) {
            if (seg_lo[sg] >= seg_hi[sg]) continue;
            if (sg == 1 && seg_lo[0] < seg_hi[0]) {
                // switch books: every decode thread is done with the first one (barrier among the decode warps only)
                asm volatile("bar.sync 1, %0;" ::"n"(GR_DECODE_WARPS * 32) : "memory");
                const uint4* t1 = (const uint4*)m.table2;
                uint4* dst = (uint4*)smem;
                for (int i = tid; i < 4096; i += GR_DECODE_WARPS * 32) dst[i] = __ldg(t1 + i);
                asm volatile("bar.sync 1, %0;" ::"n"(GR_DECODE_WARPS * 32) : "memory");
            }
            uint32_t wa = 0, wb = 0, wc = 0, na = 0, nb = 0, nc = 0;
            auto load_tags = [&](int kb, uint32_t& a, uint32_t& b, uint32_t& c) {
                a = b = c = 0;
                if (live && kb < seg_hi[sg]) {
                    const uint32_t* p = wp + (int64_t)kb * 3 * m.Rpad;
                    a = __ldg(p); b = __ldg(p + m.Rpad); c = __ldg(p + 2 * (int64_t)m.Rpad);
                }
            };
            load_tags(seg_lo[sg] + kbs, wa, wb, wc);
            for (int kb = seg_lo[sg]; kb < seg_hi[sg]; kb += GR_KBS, it++) {
                const int s = it % GT_STAGES;
                load_tags(kb + GR_KBS + kbs, na, nb, nc);
                wait(empty(s), ((it / GT_STAGES) & 1) ^ 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");      // the MMAs that read this TMEM stage are complete
                if (kb + kbs < seg_hi[sg]) {
                    uint32_t off[8];
                    off[0] = (wa << 4) & 0xFFF0u;
                    off[1] = (wa >> 8) & 0xFFF0u;
                    off[2] = __funnelshift_r(wa, wb, 20) & 0xFFF0u;
                    off[3] = wb & 0xFFF0u;
                    off[4] = (wb >> 12) & 0xFFF0u;
                    off[5] = __funnelshift_r(wb, wc, 24) & 0xFFF0u;
                    off[6] = (wc >> 4) & 0xFFF0u;
                    off[7] = (wc >> 16) & 0xFFF0u;
                    uint4 cw[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) cw[c] = cbl_lds128(sbase + off[c]);
                    // the row's 64 values of this k-block = 32 consecutive 32-bit columns of its TMEM lane
                    tmem_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(GT_A_COL0 + s * GT_A_STAGE_COLS + kbs * 32), cw);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(s));
                wa = na; wb = nb; wc = nc;
            }
        }
        // ---------------- epilogue: decode warps 0..3 read TMEM lanes (= W rows) 32 w ..; columns = tokens
        if (warp < 4) {
            wait(tmem_full, 0);
            const bool ok = *(volatile int*)&s_abort == 0;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = r0 + warp * 32 + lane;
            if (ok) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < m.R) {
                    if (P.ksplit == 1) {
                        const float rs = __half2float(__ldg((const __half*)m.row_scale + r));
#pragma unroll 4
                        for (int n = 0; n < GR_NMAX; n++)
                            if (n < ntok) cbl_store_out(P.y[mi], ydtype, (int64_t)n * ldy + r, __uint_as_float(v[n]) * xinv[n] * rs);
                    } else {
                        float* acc = P.acc[mi] + r;
#pragma unroll 4
                        for (int n = 0; n < GR_NMAX; n++)
                            if (n < ntok) atomicAdd(acc + (int64_t)n * m.Rpad, __uint_as_float(v[n]));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    if (warp == GR_DECODE_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// k-split launches: y[n][r] = round(sum * token scale * row scale); the sums are left zero.  blockIdx.y = token,
// blockIdx.z = matrix of the group.
__global__ void __launch_bounds__(256) k_rows_finish(const __grid_constant__ GRLaunch P, const float* __restrict__ xinv, int ydtype, int64_t ldy) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const cbl_l8& m = P.m[blockIdx.z];
    const int r = blockIdx.x * blockDim.x + threadIdx.x, n = blockIdx.y;
    if (r >= m.R) return;
    float* a = P.acc[blockIdx.z] + (int64_t)n * m.Rpad + r;
    const float v = __ldcg(a);
    __stcg(a, 0.f);
    cbl_store_out(P.y[blockIdx.z], ydtype, (int64_t)n * ldy + r, v * xinv[n] * __half2float(((const __half*)m.row_scale)[r]));
}

// ------------------------------------------------------------------------------------ two-phase variant for many tokens
//
// The fused kernels above decode every weight tile once per 256 (or 512) tokens; their shared-memory pipe
// carries the codeword gathers, the B-tile stores, the activation tiles and the tensor cores' operand
// reads, and saturates before the tensor pipe does.  From about a thousand tokens on it is cheaper to
// decode the matrix ONCE into a 16-bit scratch (k_decode_raw: raw codewords, or the sum of the two books'
// codewords, column orders undone) and to run a plain TMA-fed tcgen05 GEMM over it (k_gemm_dense: both
// operands arrive by TMA, nothing but the tensor cores reads shared memory).  Row scales and the tokens'
// power-of-two scales are applied in the epilogue exactly as in the fused kernel.  The scratch also
// serves matrices with several column orders, which the fused kernels do not execute.
constexpr int GD_STAGES = 3;
constexpr int GD_STAGE_BYTES = 2 * GM_A_BYTES + GM_B_BYTES;                 // 256 tokens + 256 rows of one k-block: 64 KB
constexpr int GD_SMEM = GD_STAGES * GD_STAGE_BYTES + 1024;                  // + slack to align the ring to 1024 bytes
constexpr int GD_EPI_WARPS = 8, GD_THREADS = (GD_EPI_WARPS + 2) * 32;

__global__ void __launch_bounds__(GD_THREADS, 1)
k_gemm_dense(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, cbl_l8 m, const float* __restrict__ xinv,
             int ntok, void* __restrict__ y, int ydtype, int64_t ldy, int vec_ok, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2 * GD_STAGES + 1];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // token tiles vary fastest across the grid: blocks that run together share weight rows in L2
    const int r0 = blockIdx.y * GM_BN, tok0 = blockIdx.x * GM_BM;
    const int nkb = (m.C + GM_BK - 1) / GM_BK;
    const uint32_t sbase = (cbl_smem_u32(smem_raw) + 1023u) & ~1023u, bar0 = cbl_smem_u32(s_bar);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (GD_STAGES + s); };
    const uint32_t tmem_full = bar0 + 8u * (2 * GD_STAGES);
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < GD_STAGES; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == GD_EPI_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == GD_EPI_WARPS) {
        if (lane == 0) {                                      // TMA producer: activations (2 x 128 tokens) and weights (256 rows)
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % GD_STAGES;
                if (!mbar_wait(empty(s), ((kb / GD_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
                mbar_expect_tx(full(s), GD_STAGE_BYTES);
                const uint32_t dst = sbase + s * GD_STAGE_BYTES;
                tma_load_2d(dst, &xmap, kb * GM_BK, tok0, full(s));
                tma_load_2d(dst + GM_A_BYTES, &xmap, kb * GM_BK, tok0 + 128, full(s));
                tma_load_2d(dst + 2 * GM_A_BYTES, &wmap, kb * GM_BK, r0, full(s));
            }
        }
    } else if (warp == GD_EPI_WARPS + 1) {
        if (lane == 0) {                                      // MMA issuer
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(GM_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % GD_STAGES;
                if (!mbar_wait(full(s), (kb / GD_STAGES) & 1)) { s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = sbase + s * GD_STAGE_BYTES, b_addr = a_addr + 2 * GM_A_BYTES;
#pragma unroll
                for (int tb = 0; tb < 2; tb++) {
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; kk++) {
                        const uint64_t da = umma_desc_sw128(a_addr + tb * GM_A_BYTES + kk * 32);
                        const uint64_t db = umma_desc_sw128(b_addr + kk * 32);
                        umma_f16(tmem + tb * GM_BN, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                }
                umma_commit(empty(s));
            }
            umma_commit(tmem_full);
        }
    } else {
        const bool ok = mbar_wait(tmem_full, 0);
        if (!ok) s_abort = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3, tb = warp >> 2;
        const int tok = tok0 + tb * 128 + q * 32 + lane;
        const float tsc = (tok < ntok) ? xinv[tok] : 0.f;
        if (ok) {
            for (int c0 = 0; c0 < GM_BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(tb * GM_BN + c0), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                gemm_store_row32(v, tok, ntok, r0 + c0, m, tsc, y, ydtype, ldy, vec_ok);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    if (warp == GD_EPI_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// The same GEMM on pairs of thread blocks, persistent, with the epilogue overlapped: a cluster of two blocks
// computes 256-token x 256-row tiles with tcgen05.mma.cta_group::2 (each block holds 128 tokens of the
// activations and 128 rows of the weights per k-block, so the traffic from L2 per MMA cycle is the one of a
// 256 x 256 tile although a block only accumulates 128 x 256).  A block's accumulator takes 256 of the 512
// tensor-memory columns: two buffers alternate, the epilogue warps drain one while the MMAs fill the other.
// Barriers: "full" (leader block; TMA bytes of both blocks), "empty" and "accumulator full" (each block;
// multicast commits from the leader), "accumulator empty" (leader; one arrival per epilogue warp of both blocks).
constexpr int G3_STAGES = 4;              // 128 KB: leaves room for a decode block of the NEXT matrix on the same SM
constexpr int G3_STAGE_BYTES = GM_A_BYTES + 128 * GM_BK * 2;                // 128 tokens + 128 rows of one k-block: 32 KB
constexpr int G3_SMEM = G3_STAGES * G3_STAGE_BYTES + 1024;
constexpr int G3_EPI_WARPS = 8, G3_THREADS = (G3_EPI_WARPS + 2) * 32;

__global__ void __launch_bounds__(G3_THREADS, 1)
k_gemm_dense_2sm(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, cbl_l8 m, const float* __restrict__ xinv,
                 int ntok, void* __restrict__ y, int ydtype, int64_t ldy, int vec_ok, unsigned int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2 * G3_STAGES + 4];   // full, empty per stage; acc_full[2], acc_empty[2]
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // a decode kernel of the next matrix (launched with programmatic serialization) may share the SMs with this GEMM
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int nkb = (m.C + GM_BK - 1) / GM_BK;
    const int ntt = (ntok + 255) / 256, nrt = (m.R + GM_BN - 1) / GM_BN, ntiles = ntt * nrt;
    const int cluster = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
    const uint32_t sbase = (cbl_smem_u32(smem_raw) + 1023u) & ~1023u, bar0 = cbl_smem_u32(s_bar);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (G3_STAGES + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * G3_STAGES + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * G3_STAGES + 2 + b); };
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < G3_STAGES; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 2 * G3_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == G3_EPI_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbl_smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                        // both blocks' barriers and tensor memory exist
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp == G3_EPI_WARPS) {
        if (lane == 0) {                                      // TMA producer: this block's 128 tokens and 128 weight rows
            int it = 0;
            for (int t = cluster; t < ntiles && !s_abort; t += nclusters) {
                const int tok0 = (t % ntt) * 256 + (int)rank * 128, r0 = (t / ntt) * GM_BN + (int)rank * 128;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % G3_STAGES;
                    if (!mbar_wait(empty(s), ((it / G3_STAGES) & 1) ^ 1)) { s_abort = 1; break; }
                    if (rank == 0) mbar_expect_tx(full(s), 2 * G3_STAGE_BYTES);
                    const uint32_t dst = sbase + s * G3_STAGE_BYTES;
                    const uint32_t lead_bar = mapa_u32(full(s), 0);
                    tma_load_2d_2sm(dst, &xmap, kb * GM_BK, tok0, lead_bar);
                    tma_load_2d_2sm(dst + GM_A_BYTES, &wmap, kb * GM_BK, r0, lead_bar);
                }
            }
        }
    } else if (warp == G3_EPI_WARPS + 1) {
        if (lane == 0 && rank == 0) {                         // MMA issuer (leader block)
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(GM_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int it = 0, li = 0;
            for (int t = cluster; t < ntiles && !s_abort; t += nclusters, li++) {
                const int buf = li & 1;
                if (!mbar_wait(acc_empty(buf), ((li >> 1) & 1) ^ 1)) { s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int s = it % G3_STAGES;
                    if (!mbar_wait(full(s), (it / G3_STAGES) & 1)) { s_abort = 1; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = sbase + s * G3_STAGE_BYTES, b_addr = a_addr + GM_A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; kk++)
                        umma_f16_2sm(tmem + buf * GM_BN, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc,
                                     (kb | kk) ? 1u : 0u);
                    umma_commit_2sm(empty(s));
                }
                umma_commit_2sm(acc_full(buf));
            }
        }
    } else {
        // epilogue: warp w drains TMEM lanes 32 (w % 4).., columns 128 (w / 4).. of the tile's buffer
        const int q = warp & 3, ch = warp >> 2;
        int li = 0;
        for (int t = cluster; t < ntiles; t += nclusters, li++) {
            const int buf = li & 1;
            if (!mbar_wait(acc_full(buf), (li >> 1) & 1)) { s_abort = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int tok = (t % ntt) * 256 + (int)rank * 128 + q * 32 + lane, r0 = (t / ntt) * GM_BN;
            const float tsc = (tok < ntok) ? xinv[tok] : 0.f;
            for (int c0 = ch * 128; c0 < ch * 128 + 128; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * GM_BN + c0), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                gemm_store_row32(v, tok, ntok, r0 + c0, m, tsc, y, ydtype, ldy, vec_ok);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(acc_empty(buf), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort && tid == 0) atomicExch(status, 1u);
    cluster_sync_all();                                        // the peer no longer reads or signals this block's memory
    if (warp == G3_EPI_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// Raw 16-bit decode of a packed matrix (d = 8, 12-bit tags): out[r, col] = fp16(A[a] (+ B[b])) without the row
// scale, col = the original column (column orders undone).  A warp walks one row 256 chunks at a time, lane l
// taking chunks l, l + 32, ...: the 16-byte codewords of a warp-wide store are contiguous.  The book(s) sit in
// shared memory.  One block of 512 threads per SM; it is launched with programmatic serialization and waits
// for its predecessors only at its END, so that it decodes the next matrix beside a running GEMM (which
// leaves shared memory for it) while everything after it still sees the stream's order.
constexpr int DR_THREADS = 512;            // x 56 registers: fits beside the GEMM's 320 threads x 104 registers
template <int BOOKS, bool PERM>
__global__ void __maxnreg__(56) k_decode_raw(cbl_packed m, __half* __restrict__ out, int64_t ld) {
    extern __shared__ __align__(16) unsigned char dsm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    {
        uint4* dst = (uint4*)dsm;
        const uint4* t0 = (const uint4*)m.table;
        for (int i = tid; i < 4096; i += DR_THREADS) dst[i] = __ldg(t0 + i);
        if (BOOKS == 2) {
            const uint4* t1 = (const uint4*)m.table2;
            for (int i = tid; i < 4096; i += DR_THREADS) dst[4096 + i] = __ldg(t1 + i);
        }
    }
    __syncthreads();
    const uint32_t sb = cbl_smem_u32(dsm);
    const int nch = m.C >> 3;
    auto tag_of = [&](const int32_t* rw, int j) {
        const uint32_t bit = 12u * (uint32_t)j, w = bit >> 5, sh = bit & 31u;
        const uint32_t lo = (uint32_t)__ldg(rw + w);
        const uint32_t hi = (sh > 20u && (int)(w + 1) < m.W) ? (uint32_t)__ldg(rw + w + 1) : 0u;
        return (__funnelshift_r(lo, hi, sh) & 0xFFFu) << 4;
    };
    for (int r = blockIdx.x * (DR_THREADS / 32) + warp; r < m.R; r += gridDim.x * (DR_THREADS / 32)) {
        const int32_t* rw = m.tags + (int64_t)r * m.W;
        const int32_t* rw2 = BOOKS == 2 ? m.tags2 + (int64_t)r * m.W : nullptr;
        const int32_t* perm = PERM ? m.perms + (int64_t)m.row_mask[r] * m.C : nullptr;
        __half* orow = out + (int64_t)r * ld;
        for (int j0 = 0; j0 < nch; j0 += 256) {
            uint4 cw[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = j0 + 32 * i + lane;
                cw[i] = make_uint4(0, 0, 0, 0);
                if (j < nch) cw[i] = cbl_lds128(sb + tag_of(rw, j));
            }
            if (BOOKS == 2) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int j = j0 + 32 * i + lane;
                    if (j < nch) {
                        const uint4 o = cbl_lds128(sb + 65536u + tag_of(rw2, j));
                        __half2* a = (__half2*)&cw[i];
                        const __half2* b = (const __half2*)&o;
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float2 fa = __half22float2(a[e]), fb = __half22float2(b[e]);
                            a[e] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = j0 + 32 * i + lane;
                if (j < nch) {
                    if (!PERM) {
                        *(uint4*)(orow + j * 8) = cw[i];
                    } else {
                        const __half* hv = (const __half*)&cw[i];
#pragma unroll
                        for (int e = 0; e < 8; e++) orow[__ldg(perm + j * 8 + e)] = hv[e];
                    }
                }
            }
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");          // later kernels that wait for this one also wait for its predecessors
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
    }
    return fn;
}

}  // namespace

// Staging of the activations for cbl_gemm_l8: fp16 [Mpad8][Cpad512] followed by fp32 [Mpad8] inverse scales
// (the layout cbl_prep_x writes for one column order).
extern "C" size_t cbl_gemm_stage_bytes(int32_t ntok, int32_t C) { return cbl_prep_x_bytes(ntok, C, 1); }

static int gemm_l8_impl(const cbl_l8* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                        void* stage, void* workspace, cbl_stream s, int two_sm) {
    if (!m || !m->words || !m->table || !m->row_scale || !x || !y || !stage || !workspace) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && (!m->table2 || ((uintptr_t)m->table2 % 16))) return CBL_EINVAL;
    if (m->books == 2 && two_sm) return CBL_EUNSUPPORTED;      // the two-SM variant executes one book
    if (m->rot != 0 || m->R <= 0 || m->C <= 0 || m->C % 8 || m->Rpad != (m->R + 3) / 4 * 4 || m->ntile != m->books * cbl_ceil_div(m->C / 8, 8)) return CBL_EINVAL;
    if (ntok <= 0 || ldx < m->C || ldy < m->R) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (((uintptr_t)stage % 16) || ((uintptr_t)m->table % 16) || ((uintptr_t)workspace % 4)) return CBL_EINVAL;
    cudaStream_t st = (cudaStream_t)s;
    int rc = cbl_prep_x(x, xdtype, ntok, m->C, ldx, nullptr, 1, stage, s);
    if (rc) return rc;
    const int Mpad = (ntok + 7) / 8 * 8, Cpad = (m->C + 511) / 512 * 512;
    encode_tiled_fn enc = get_encode();
    if (!enc) return CBL_ECUDA;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)Cpad, (cuuint64_t)Mpad};
    const cuuint64_t strides[1] = {(cuuint64_t)Cpad * 2};
    const cuuint32_t box[2] = {GM_BK, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, stage, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        g_cbl_last_cuda_error = (int)cr;
        return CBL_ECUDA;
    }
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemm_l8, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
        attr_set[dev] = true;
    }
    const float* xinv = (const float*)((const __half*)stage + (int64_t)Mpad * Cpad);
    const int esz = ydtype == CBL_F32 ? 4 : 2;
    const int vec_ok = ((uintptr_t)y % 16 == 0) && ((ldy * esz) % 16 == 0) && ((uintptr_t)m->row_scale % 16 == 0);
    if (two_sm && ntok > GM_BM) {
        static bool attr2_set[64] = {};
        if (dev >= 0 && dev < 64 && !attr2_set[dev]) {
            CBL_CUDA(cudaFuncSetAttribute(k_gemm_l8_2sm, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM));
            attr2_set[dev] = true;
        }
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * cbl_ceil_div(m->R, GM_BN), cbl_ceil_div(ntok, 512));
        cfg.blockDim = dim3(G2_THREADS);
        cfg.dynamicSmemBytes = G2_SMEM;
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_l8_2sm, map, *m, xinv, (int)ntok, y, ydtype, ldy, vec_ok, (unsigned int*)workspace));
        return cbl_check_launch();
    }
    dim3 grid(cbl_ceil_div(m->R, GM_BN), cbl_ceil_div(ntok, GM_BM));
    k_gemm_l8<<<grid, GM_THREADS, GM_SMEM, st>>>(map, *m, xinv, ntok, y, ydtype, ldy, vec_ok, (unsigned int*)workspace);
    return cbl_check_launch();
}

extern "C" int cbl_gemm_l8(const cbl_l8* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                           void* stage, void* workspace, cbl_stream s) {
    return gemm_l8_impl(m, x, xdtype, ntok, ldx, y, ydtype, ldy, stage, workspace, s, 0);
}

// Same product with pairs of thread blocks on tcgen05.mma.cta_group::2 (each block decodes half of the
// weight tile).  Token counts up to 256 run the one-block kernel.
extern "C" int cbl_gemm_l8_2sm(const cbl_l8* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                               void* stage, void* workspace, cbl_stream s) {
    return gemm_l8_impl(m, x, xdtype, ntok, ldx, y, ydtype, ldy, stage, workspace, s, 1);
}

// ---- two-phase variant: host side
extern "C" size_t cbl_dense_scratch_bytes(int32_t R, int32_t C) {
    if (R < 0 || C < 0) return 0;
    return (size_t)R * ((size_t)(C + 7) / 8 * 8) * 2;
}

static int decode_raw_impl(const cbl_packed* m, void* out, int32_t C_out, cbl_stream s) {
    if (!m || !m->tags || !m->table || !out || ((uintptr_t)out % 16) || ((uintptr_t)m->table % 16)) return CBL_EINVAL;
    if (C_out < m->C || (C_out > m->C && m->M <= 1)) return CBL_EINVAL;      // a wider output only makes sense with column orders
    if (m->d != 8 || m->bits != 12 || m->G != 1) return CBL_EUNSUPPORTED;
    if (m->R < 0 || m->C <= 0 || m->C % 8 || (int64_t)m->W * 32 < (int64_t)(m->C / 8) * 12) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && (!m->tags2 || !m->table2 || ((uintptr_t)m->table2 % 16))) return CBL_EINVAL;
    if (m->M > 1 && (!m->row_mask || !m->perms)) return CBL_EINVAL;
    if (m->R == 0) return CBL_OK;
    const int64_t ld = ((int64_t)C_out + 7) / 8 * 8;
    const size_t smem = (size_t)65536 * m->books;
    int grid = cbl_sm_count();
    if (grid > cbl_ceil_div(m->R, DR_THREADS / 32)) grid = cbl_ceil_div(m->R, DR_THREADS / 32);
    const cudaStream_t st = (cudaStream_t)s;
    static bool attr_set[64][4] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(DR_THREADS);
    cfg.dynamicSmemBytes = smem;
#define CBL_RAW(BK, PM, SLOT)                                                                                              \
    do {                                                                                                                   \
        if (dev >= 0 && dev < 64 && !attr_set[dev][SLOT]) {                                                                \
            CBL_CUDA(cudaFuncSetAttribute(k_decode_raw<BK, PM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * BK)); \
            attr_set[dev][SLOT] = true;                                                                                    \
        }                                                                                                                  \
        CBL_CUDA(cudaLaunchKernelEx(&cfg, k_decode_raw<BK, PM>, *m, (__half*)out, ld));                                    \
    } while (0)
    if (m->books == 1 && m->M == 1) CBL_RAW(1, false, 0);
    else if (m->books == 1) CBL_RAW(1, true, 1);
    else if (m->M == 1) CBL_RAW(2, false, 2);
    else CBL_RAW(2, true, 3);
#undef CBL_RAW
    return cbl_check_launch();
}

extern "C" int cbl_decode_raw(const cbl_packed* m, void* out, cbl_stream s) { return decode_raw_impl(m, out, m ? m->C : 0, s); }

// The same for a column shard of a matrix with several column orders, whose orders name positions of the FULL
// activation vector (C_out of them): the scratch row is C_out wide and the shard's weights land at their positions.
extern "C" int cbl_decode_raw_wide(const cbl_packed* m, void* out, int32_t C_out, cbl_stream s) { return decode_raw_impl(m, out, C_out, s); }

extern "C" int cbl_gemm_dense(const void* w16, int32_t R, int32_t C, const void* row_scale, const void* x, int xdtype, int32_t ntok,
                              int64_t ldx, void* y, int ydtype, int64_t ldy, void* stage, void* workspace, cbl_stream s) {
    if (!w16 || !row_scale || !x || !y || !stage || !workspace) return CBL_EINVAL;
    if (R <= 0 || C <= 0 || C % 8 || ntok <= 0 || ldx < C || ldy < R) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (((uintptr_t)stage % 16) || ((uintptr_t)w16 % 16) || ((uintptr_t)workspace % 4)) return CBL_EINVAL;
    const cudaStream_t st = (cudaStream_t)s;
    int rc = cbl_prep_x(x, xdtype, ntok, C, ldx, nullptr, 1, stage, s);
    if (rc) return rc;
    const int Mpad = (ntok + 7) / 8 * 8, Cpad = (C + 511) / 512 * 512;
    encode_tiled_fn enc = get_encode();
    if (!enc) return CBL_ECUDA;
    CUtensorMap xmap, wmap;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)Cpad, (cuuint64_t)Mpad};
        const cuuint64_t strides[1] = {(cuuint64_t)Cpad * 2};
        const cuuint32_t box[2] = {GM_BK, 128};
        CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, stage, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { g_cbl_last_cuda_error = (int)cr; return CBL_ECUDA; }
    }
    {
        // columns beyond C and rows beyond R are outside the map: TMA fills them with zeros
        const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)R};
        const cuuint64_t strides[1] = {(cuuint64_t)((C + 7) / 8 * 8) * 2};
        const cuuint32_t box[2] = {GM_BK, GM_BN};
        CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)w16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { g_cbl_last_cuda_error = (int)cr; return CBL_ECUDA; }
    }
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemm_dense, cudaFuncAttributeMaxDynamicSharedMemorySize, GD_SMEM));
        attr_set[dev] = true;
    }
    cbl_l8 m = {};
    m.R = R;
    m.C = C;
    m.row_scale = row_scale;
    const float* xinv = (const float*)((const __half*)stage + (int64_t)Mpad * Cpad);
    const int esz = ydtype == CBL_F32 ? 4 : 2;
    const int vec_ok = ((uintptr_t)y % 16 == 0) && ((ldy * esz) % 16 == 0) && ((uintptr_t)row_scale % 16 == 0);
#ifdef CBL_DENSE_1SM
    const int variant = 1;                                    // build option: the one-block kernel (for comparisons)
#else
    const int variant = 2;
#endif
    if (variant == 2) {
        // box of the pair kernel: 128 tokens / 128 weight rows per block
        {
            const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)R};
            const cuuint64_t strides[1] = {(cuuint64_t)((C + 7) / 8 * 8) * 2};
            const cuuint32_t box[2] = {GM_BK, 128};
            CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)w16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) { g_cbl_last_cuda_error = (int)cr; return CBL_ECUDA; }
        }
        static bool attr3_set[64] = {};
        if (dev >= 0 && dev < 64 && !attr3_set[dev]) {
            CBL_CUDA(cudaFuncSetAttribute(k_gemm_dense_2sm, cudaFuncAttributeMaxDynamicSharedMemorySize, G3_SMEM));
            attr3_set[dev] = true;
        }
        const int ntiles = cbl_ceil_div(R, GM_BN) * cbl_ceil_div(ntok, 256);
        int nclusters = cbl_sm_count() / 2;
        if (nclusters > ntiles) nclusters = ntiles;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * nclusters);
        cfg.blockDim = dim3(G3_THREADS);
        cfg.dynamicSmemBytes = G3_SMEM;
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_dense_2sm, xmap, wmap, m, xinv, (int)ntok, y, ydtype, ldy, vec_ok, (unsigned int*)workspace));
        return cbl_check_launch();
    }
    dim3 grid(cbl_ceil_div(ntok, GM_BM), cbl_ceil_div(R, GM_BN));
    k_gemm_dense<<<grid, GD_THREADS, GD_SMEM, st>>>(xmap, wmap, m, xinv, ntok, y, ydtype, ldy, vec_ok, (unsigned int*)workspace);
    return cbl_check_launch();
}

// ---- up to 32 tokens: host side
extern "C" int32_t cbl_gemm_rows_max_tokens(void) { return GR_NMAX; }

extern "C" size_t cbl_gemm_rows_workspace_bytes(int32_t sum_rows_padded) {
    if (sum_rows_padded < 0) return 0;
    return (size_t)GR_NMAX * (size_t)sum_rows_padded * 4 + 16;
}

extern "C" int cbl_gemm_rows_multi(const cbl_l8* mats, int32_t n, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* const* ys, int ydtype,
                                   int64_t ldy, void* stage, void* workspace, cbl_stream s) {
    if (!mats || !ys || !x || !stage || !workspace || n < 1) return CBL_EINVAL;
    if (n > GR_MAX_GROUP || ntok > GR_NMAX) return CBL_EUNSUPPORTED;
    if (ntok < 1) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (((uintptr_t)stage % 16) || ((uintptr_t)workspace % 16)) return CBL_EINVAL;
    GRLaunch P;
    P.n = 0;
    P.tile0[0] = 0;
    size_t off = 0;
    for (int i = 0; i < n; i++) {
        const cbl_l8* m = mats + i;
        if (!m->words || !m->table || !m->row_scale || !ys[i]) return CBL_EINVAL;
        if (m->books != 1 && m->books != 2) return CBL_EINVAL;
        if (m->books == 2 && (!m->table2 || ((uintptr_t)m->table2 % 16))) return CBL_EINVAL;
        if (m->rot != 0 || m->R < 0 || m->C <= 0 || m->C % 8 || m->Rpad != (m->R + 3) / 4 * 4 || m->ntile != m->books * cbl_ceil_div(m->C / 8, 8)) return CBL_EINVAL;
        if (m->C != mats[0].C || m->books != mats[0].books || ldx < m->C || ldy < m->R || ((uintptr_t)m->table % 16)) return CBL_EINVAL;
        if (m->R == 0) continue;
        P.m[P.n] = *m;
        P.acc[P.n] = (float*)((char*)workspace + off);
        P.y[P.n] = ys[i];
        P.tile0[P.n + 1] = P.tile0[P.n] + cbl_ceil_div(m->R, GR_ROWS);
        off += (size_t)GR_NMAX * m->Rpad * 4;
        P.n++;
    }
    if (P.n == 0) return CBL_OK;
    unsigned int* status = (unsigned int*)((char*)workspace + off);
    const int C = mats[0].C, nkb = mats[0].ntile;
    const cudaStream_t st = (cudaStream_t)s;
    int rc = cbl_prep_x(x, xdtype, ntok, C, ldx, nullptr, 1, stage, s);
    if (rc) return rc;
    const int Mpad = (ntok + 7) / 8 * 8, Cpad = (C + 511) / 512 * 512;
    P.npad = ntok <= 16 ? 16 : 32;
    // few row tiles: split along k so that about every SM gets a block, at least two stages of k-blocks per part
    const int tiles = P.tile0[P.n];
    int ksplit = 1;
    if (tiles * 2 <= cbl_sm_count()) {
        ksplit = cbl_sm_count() / tiles;
        const int most = nkb / (2 * GR_KBS);
        if (ksplit > most) ksplit = most;
        if (ksplit < 1) ksplit = 1;
    }
    P.ksplit = ksplit;
    encode_tiled_fn enc = get_encode();
    if (!enc) return CBL_ECUDA;
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)Cpad, (cuuint64_t)Mpad};
    const cuuint64_t strides[1] = {(cuuint64_t)Cpad * 2};
    const cuuint32_t box[2] = {GM_BK, (cuuint32_t)P.npad};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, stage, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) { g_cbl_last_cuda_error = (int)cr; return CBL_ECUDA; }
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemm_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, GR_SMEM));
        CBL_CUDA(cudaFuncSetAttribute(k_gemm_rows_ta, cudaFuncAttributeMaxDynamicSharedMemorySize, GT_SMEM));
        attr_set[dev] = true;
    }
#ifdef CBL_ROWS_SMEM_A
    const int ta = 0;                                          // build option: the A tile through shared memory (comparisons)
#else
    const int ta = 1;
#endif
    const float* xinv = (const float*)((const __half*)stage + (int64_t)Mpad * Cpad);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(tiles, ksplit);
    cfg.blockDim = dim3(GR_THREADS);
    cfg.dynamicSmemBytes = ta ? GT_SMEM : GR_SMEM;
    if (ta) CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_rows_ta, xmap, P, xinv, (int)ntok, ydtype, ldy, status));
    else CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_rows, xmap, P, xinv, (int)ntok, ydtype, ldy, status));
    if (ksplit > 1) {
        int maxR = 0;
        for (int i = 0; i < P.n; i++) maxR = maxR > P.m[i].R ? maxR : P.m[i].R;
        cfg.gridDim = dim3(cbl_ceil_div(maxR, 256), ntok, P.n);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        CBL_CUDA(cudaLaunchKernelEx(&cfg, k_rows_finish, P, xinv, ydtype, ldy));
    }
    return cbl_check_launch();
}

