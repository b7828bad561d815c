// Decode-time products straight from the packed tags (d = 8, 12-bit tags, 4096-entry fp16 books).
//
//   cbl_gemv_t16: batch <= 64.  The 64 KB book (128 KB for two summed books) lives in shared memory;
//                 a 16-byte codeword read lands directly in an mma.sync A fragment, the activations
//                 are the B fragment, accumulation is fp32.  Bound by shared-memory gather rate
//                 (random 16-byte reads), not by HBM.
//   cbl_gemv_l8:  batch 1.  Per tile of 8 chunk columns the block first computes the table
//                 T[c][e] = <book[e], x_c> for all 4096 codewords (mma.sync m16n8k8, fp32 results in
//                 shared memory); every weight chunk then costs one 4-byte shared-memory read and
//                 one add.  Row sums are accumulated across tiles with vector reductions in L2 and
//                 finished (row scale, output rounding, re-zeroing) by a second small kernel.
#include <utility>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>
#include "cbl_common.cuh"

// ------------------------------------------------------------------------------------ activations
// xp holds fp16 [M][Bpad][Cpad] followed by fp32 [M][Bpad] inverse scales: each batch row is multiplied
// by a power of two that brings its largest magnitude to [2^13, 2^14) before the fp16 conversion, so
// that neither bf16/fp32 outliers overflow nor tiny activations underflow; the product kernel
// multiplies the fp32 result by the inverse.
extern "C" size_t cbl_prep_x_bytes(int32_t B, int32_t C, int32_t M) {
    if (B <= 0 || C <= 0 || M <= 0) return 0;
    size_t Bpad = ((size_t)B + 7) / 8 * 8, Cpad = ((size_t)C + 511) / 512 * 512;
    return (size_t)M * Bpad * Cpad * 2 + (size_t)M * Bpad * 4;
}

// Power-of-two exponent k such that |v| * 2^-k < 2^14 for the largest magnitude mx (k may be negative).
__device__ __forceinline__ int cbl_scale_exp(float mx) {
    if (!(mx > 0.f) || !(mx < 3.0e38f)) return 0;
    int k = ilogbf(mx) - 13;
    return k < -100 ? -100 : (k > 110 ? 110 : k);
}

__global__ void __launch_bounds__(256) k_prep_x(const void* __restrict__ x, int xdtype, int B, int C, int64_t ldx,
                                                const int32_t* __restrict__ perms, int Bpad, int Cpad, __half* __restrict__ xp,
                                                float* __restrict__ xinv) {
    __shared__ float s_max[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x % Bpad, m = blockIdx.x / Bpad;
    __half* dst = xp + (int64_t)blockIdx.x * Cpad;
    float mx = 0.f;
    if (b < B)
        for (int c = threadIdx.x; c < C; c += 256) mx = fmaxf(mx, fabsf(cbl_load_in(x, xdtype, (int64_t)b * ldx + c)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = s_max[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, s_max[i]);
    const int k = cbl_scale_exp(mx);
    const float sc = ldexpf(1.f, -k);
    if (threadIdx.x == 0) xinv[blockIdx.x] = ldexpf(1.f, k);
    for (int c = threadIdx.x; c < Cpad; c += 256) {
        float v = 0.f;
        if (b < B && c < C) {
            int src = perms ? perms[(int64_t)m * C + c] : c;
            v = cbl_load_in(x, xdtype, (int64_t)b * ldx + src) * sc;
        }
        dst[c] = __float2half_rn(v);
    }
}

extern "C" int cbl_prep_x(const void* x, int xdtype, int32_t B, int32_t C, int64_t ldx, const int32_t* perms, int32_t M,
                          void* xp, cbl_stream s) {
    if (!x || !xp || B <= 0 || C <= 0 || M <= 0 || ldx < C) return CBL_EINVAL;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if (M > 1 && !perms) return CBL_EINVAL;
    int Bpad = (B + 7) / 8 * 8, Cpad = (C + 511) / 512 * 512;
    float* xinv = (float*)((__half*)xp + (int64_t)M * Bpad * Cpad);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = (cudaStream_t)s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(M * Bpad);
    cfg.blockDim = dim3(256);
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_prep_x, x, xdtype, (int)B, (int)C, ldx, M > 1 ? perms : (const int32_t*)nullptr, Bpad, Cpad,
                                (__half*)xp, xinv));
    return cbl_check_launch();
}

#ifdef CBL_TRACE
// Debug builds only: per-block phase timestamps (ns) for offline inspection.
__device__ unsigned long long g_cbl_trace[1024 * 16];
__device__ __forceinline__ unsigned long long cbl_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define CBL_MARK(i) do { if (threadIdx.x == 0 && blockIdx.x < 1024) g_cbl_trace[blockIdx.x * 16 + (i)] = cbl_now(); } while (0)
extern "C" int cbl_trace_read(unsigned long long* host) { return (int)cudaMemcpyFromSymbol(host, g_cbl_trace, sizeof(g_cbl_trace)); }
#else
#define CBL_MARK(i) do { } while (0)
#endif

// ------------------------------------------------------------------------------------ t16 product
// Byte offset (tag * 16) of tag i of a lane's 384-bit stream held in w[0..11].
template <int I>
__device__ __forceinline__ uint32_t t16_tag_off(const uint32_t (&w)[12]) {
    constexpr int bit = 12 * I, wi = bit >> 5, sh = bit & 31;
    if constexpr (sh > 20) return __funnelshift_r(w[wi], w[wi + 1], sh - 4) & 0xFFF0u;
    else if constexpr (sh >= 4) return (w[wi] >> (sh - 4)) & 0xFFF0u;
    else return (w[wi] << (4 - sh)) & 0xFFF0u;
}

// One step = 4 chunks of each of the tile's 16 rows (two codeword reads per lane and book, two MMAs per batch
// block).  The codewords and activations of step S + 1 are requested before the MMAs of step S are issued, and
// the two MMAs of a step accumulate into separate registers (two shorter dependency chains), summed at the end.
template <int BOOKS, int NB>
struct T16Operands {
    uint4 c[BOOKS][2];
    uint4 x[NB];
};

template <int BOOKS, int NB, int S>
__device__ __forceinline__ void t16_fetch(T16Operands<BOOKS, NB>& o, const uint32_t (&w)[BOOKS][12], uint32_t tbl,
                                          const uint4* __restrict__ xrow, int64_t xstride8, int rows_left) {
    // xrow points at chunk (ss*16)*4 + t of batch row g; step S adds 4 chunks.  Lanes whose batch row does not
    // exist (padding up to a multiple of 8) feed zeros without touching memory.
#pragma unroll
    for (int nb = 0; nb < NB; nb++) o.x[nb] = (nb * 8 < rows_left) ? __ldg(xrow + S * 4 + nb * xstride8) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int bk = 0; bk < BOOKS; bk++) {
        o.c[bk][0] = cbl_lds128(tbl + bk * 65536u + t16_tag_off<2 * S>(w[bk]));
        o.c[bk][1] = cbl_lds128(tbl + bk * 65536u + t16_tag_off<2 * S + 1>(w[bk]));
    }
}

template <int BOOKS, int NB, int S>
__device__ __forceinline__ void t16_step(float (&acc)[2][NB][4], T16Operands<BOOKS, NB>& cur, const uint32_t (&w)[BOOKS][12], uint32_t tbl,
                                         const uint4* __restrict__ xrow, int64_t xstride8, int rows_left) {
    T16Operands<BOOKS, NB> nxt;
    if constexpr (S + 1 < 16) t16_fetch<BOOKS, NB, S + 1>(nxt, w, tbl, xrow, xstride8, rows_left);
#pragma unroll
    for (int bk = 0; bk < BOOKS; bk++) {
        const uint4 c0 = cur.c[bk][0], c1 = cur.c[bk][1];
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
            cbl_mma16816(acc[0][nb], c0.x, c1.x, c0.y, c1.y, cur.x[nb].x, cur.x[nb].y);
            cbl_mma16816(acc[1][nb], c0.z, c1.z, c0.w, c1.w, cur.x[nb].z, cur.x[nb].w);
        }
    }
    if constexpr (S + 1 < 16) cur = nxt;
}

template <int BOOKS, int NB, int... S>
__device__ __forceinline__ void t16_steps(float (&acc)[2][NB][4], const uint32_t (&w)[BOOKS][12], uint32_t tbl,
                                          const uint4* __restrict__ xrow, int64_t xstride8, int rows_left,
                                          std::integer_sequence<int, S...>) {
    T16Operands<BOOKS, NB> cur;
    t16_fetch<BOOKS, NB, 0>(cur, w, tbl, xrow, xstride8, rows_left);
    (t16_step<BOOKS, NB, S>(acc, cur, w, tbl, xrow, xstride8, rows_left), ...);
}

constexpr int T16_WARPS = 8;

template <int BOOKS, int NB>
__global__ void __launch_bounds__(T16_WARPS * 32) k_gemv_t16(cbl_t16 m, const __half* __restrict__ xp, int B, int Bpad, int Cpad,
                                                             void* __restrict__ y, int ydtype, int64_t ldy) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint4* s_table = (uint4*)smem;                                  // BOOKS * 4096 codewords
    float* s_red = (float*)(smem + BOOKS * 65536);                  // [warps][NB][32][4]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    CBL_MARK(0);
    {
        const uint4* t0 = (const uint4*)m.table;
        for (int i = tid; i < 4096; i += T16_WARPS * 32) s_table[i] = __ldg(t0 + i);
        if (BOOKS == 2) {
            const uint4* t1 = (const uint4*)m.table2;
            for (int i = tid; i < 4096; i += T16_WARPS * 32) s_table[4096 + i] = __ldg(t1 + i);
        }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");          // the staged activations come from the kernel before
    __syncthreads();
    CBL_MARK(1);
    int trace_it = 0;
    const uint32_t tbl = cbl_smem_u32(s_table);
    const uint4* words = (const uint4*)m.words;
    const int64_t book_stride = (int64_t)m.ntile * m.nsuper * 96;   // uint4 per book
    const int64_t xstride8 = (int64_t)8 * Cpad / 8;                 // uint4 between batch blocks of 8 rows

    for (int tile = blockIdx.x; tile < m.ntile; tile += gridDim.x) {
        const int mk = m.tile_mask ? m.tile_mask[tile] : 0;
        const float* xinv = (const float*)(xp + (int64_t)m.M * Bpad * Cpad);
        const uint4* xbase = (const uint4*)(xp + ((int64_t)mk * Bpad + g) * Cpad) + t;
        float acc[2][NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[0][nb][k] = acc[1][nb][k] = 0.f;
        uint32_t w[BOOKS][12];
        int ss = warp;
        if (ss < m.nsuper) {
#pragma unroll
            for (int bk = 0; bk < BOOKS; bk++) {
                const uint4* p = words + bk * book_stride + ((int64_t)tile * m.nsuper + ss) * 96 + lane;
#pragma unroll
                for (int q = 0; q < 3; q++) {
                    uint4 v = cbl_ldg_stream(p + 32 * q);
                    w[bk][4 * q] = v.x; w[bk][4 * q + 1] = v.y; w[bk][4 * q + 2] = v.z; w[bk][4 * q + 3] = v.w;
                }
            }
        }
        while (ss < m.nsuper) {
            const int sn = ss + T16_WARPS;
            uint32_t wn[BOOKS][12];
            if (sn < m.nsuper) {
#pragma unroll
                for (int bk = 0; bk < BOOKS; bk++) {
                    const uint4* p = words + bk * book_stride + ((int64_t)tile * m.nsuper + sn) * 96 + lane;
#pragma unroll
                    for (int q = 0; q < 3; q++) {
                        uint4 v = cbl_ldg_stream(p + 32 * q);
                        wn[bk][4 * q] = v.x; wn[bk][4 * q + 1] = v.y; wn[bk][4 * q + 2] = v.z; wn[bk][4 * q + 3] = v.w;
                    }
                }
            }
            t16_steps<BOOKS, NB>(acc, w, tbl, xbase + (int64_t)ss * 64, xstride8, B - g, std::make_integer_sequence<int, 16>{});
            if (sn < m.nsuper) {
#pragma unroll
                for (int bk = 0; bk < BOOKS; bk++)
#pragma unroll
                    for (int k = 0; k < 12; k++) w[bk][k] = wn[bk][k];
            }
            ss = sn;
        }
        if (trace_it < 4) CBL_MARK(2 + 3 * trace_it);
        // cross-warp sum in a fixed order (deterministic), row scale, output rounding
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
            *(float4*)(s_red + ((warp * NB + nb) * 32 + lane) * 4) = make_float4(acc[0][nb][0] + acc[1][nb][0], acc[0][nb][1] + acc[1][nb][1],
                                                                                 acc[0][nb][2] + acc[1][nb][2], acc[0][nb][3] + acc[1][nb][3]);
        __syncthreads();
        if (trace_it < 4) CBL_MARK(3 + 3 * trace_it);
        for (int e = tid; e < 128 * NB; e += T16_WARPS * 32) {
            int nb = e >> 7, ln = (e & 127) >> 2, k = e & 3;
            float sum = 0.f;
#pragma unroll
            for (int wq = 0; wq < T16_WARPS; wq++) sum += s_red[((wq * NB + nb) * 32 + ln) * 4 + k];
            int row = (ln >> 2) + ((k & 2) ? 8 : 0);
            int n = nb * 8 + 2 * (ln & 3) + (k & 1);
            int r = m.tile_rows[tile * 16 + row];
            if (r >= 0 && n < B) {
                float rs = __half2float(((const __half*)m.row_scale)[r]);
                cbl_store_out(y, ydtype, (int64_t)n * ldy + r, sum * xinv[mk * Bpad + n] * rs);
            }
        }
        __syncthreads();
        if (trace_it < 4) CBL_MARK(4 + 3 * trace_it);
        trace_it++;
    }
    CBL_MARK(15);
}

template <int BOOKS, int NB>
static int launch_t16(const cbl_t16* m, const void* xp, int B, void* y, int ydtype, int64_t ldy, cudaStream_t st) {
    size_t smem = (size_t)BOOKS * 65536 + (size_t)T16_WARPS * NB * 32 * 4 * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemv_t16<BOOKS, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    int per_sm = (int)(227 * 1024 / (smem + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 3) per_sm = 3;
    int grid = cbl_sm_count() * per_sm;
    if (grid > m->ntile) grid = m->ntile;
    int Bpad = NB * 8, Cpad = (m->C + 511) / 512 * 512;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(T16_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_t16<BOOKS, NB>, *m, (const __half*)xp, B, Bpad, Cpad, y, ydtype, ldy));
    return cbl_check_launch();
}

extern "C" int cbl_gemv_t16(const cbl_t16* m, const void* xp, int32_t B, void* y, int ydtype, int64_t ldy, cbl_stream s) {
    if (!m || !m->words || !m->tile_rows || !m->table || !m->row_scale || !xp || !y) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->table2) return CBL_EINVAL;
    if (m->M > 1 && !m->tile_mask) return CBL_EINVAL;
    if (B < 1 || ldy < m->R || m->C % 8 || m->nsuper != cbl_ceil_div(m->C / 8, 64)) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (B > 64) return CBL_EUNSUPPORTED;
    if (((uintptr_t)m->words % 16) || ((uintptr_t)m->table % 16) || ((uintptr_t)xp % 16)) return CBL_EINVAL;
    if (m->ntile == 0) return CBL_OK;
    cudaStream_t st = (cudaStream_t)s;
    int nb = (B + 7) / 8;
#define CBL_T16_CASE(BK, N) return launch_t16<BK, N>(m, xp, B, y, ydtype, ldy, st)
    if (m->books == 1) {
        switch (nb) {
            case 1: CBL_T16_CASE(1, 1);
            case 2: CBL_T16_CASE(1, 2);
            case 3: CBL_T16_CASE(1, 3);
            case 4: CBL_T16_CASE(1, 4);
            case 5: CBL_T16_CASE(1, 5);
            case 6: CBL_T16_CASE(1, 6);
            case 7: CBL_T16_CASE(1, 7);
            default: CBL_T16_CASE(1, 8);
        }
    } else {
        switch (nb) {
            case 1: CBL_T16_CASE(2, 1);
            case 2: CBL_T16_CASE(2, 2);
            case 3: CBL_T16_CASE(2, 3);
            case 4: CBL_T16_CASE(2, 4);
            case 5: CBL_T16_CASE(2, 5);
            case 6: CBL_T16_CASE(2, 6);
            case 7: CBL_T16_CASE(2, 7);
            default: CBL_T16_CASE(2, 8);
        }
    }
#undef CBL_T16_CASE
}

// ------------------------------------------------------------------------------------ x16 product
//
// Activation-stationary product for up to 32 tokens.  A block owns a run of 64-row blocks (at most X16_NR at a time,
// their 64 x 32 fp32 sums live in shared memory) and a run of column blocks (8 column ranges of 128 columns, one per
// warp); two blocks share an SM, so that one block's table load and output overlap the other's products.  For each column block a warp loads its activations once as MMA A fragments (tokens = M) and then walks over
// the block's rows: per 8 rows x 128 columns four 16-byte codeword reads per lane feed 8 MT MMAs (N = 8 weight
// rows), and the 8 x 16 MT results are added into the shared sums.  When the columns of a row block are split over
// several blocks (few rows, many columns) the sums go to a global fp32 accumulator and the last block to arrive
// writes the output.
constexpr int X16_WARPS = 8, X16_NR = 5, X16_ASTRIDE = 36, X16_ATILE = 64 * X16_ASTRIDE, X16_TQ = X16_WARPS * 32 / 64;

template <int MT, int RT>
__device__ __forceinline__ void x16_tile(const uint32_t (&w)[12], const uint4 (&xa)[MT][4][2], uint32_t tbl, float* __restrict__ sa, int g, int t) {
    uint4 cw[4];
#pragma unroll
    for (int j = 0; j < 4; j++) cw[j] = j == 0 ? cbl_lds128(tbl + t16_tag_off<4 * RT>(w)) : j == 1 ? cbl_lds128(tbl + t16_tag_off<4 * RT + 1>(w))
                                      : j == 2 ? cbl_lds128(tbl + t16_tag_off<4 * RT + 2>(w)) : cbl_lds128(tbl + t16_tag_off<4 * RT + 3>(w));
    float d[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) d[mt][0] = d[mt][1] = d[mt][2] = d[mt][3] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            cbl_mma16816(d[mt], xa[mt][j][0].x, xa[mt][j][1].x, xa[mt][j][0].y, xa[mt][j][1].y, cw[j].x, cw[j].y);
            cbl_mma16816(d[mt], xa[mt][j][0].z, xa[mt][j][1].z, xa[mt][j][0].w, xa[mt][j][1].w, cw[j].z, cw[j].w);
        }
    float* o = sa + (RT * 8 + 2 * t) * X16_ASTRIDE + g;
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        atomicAdd(o + mt * 16, d[mt][0]);
        atomicAdd(o + X16_ASTRIDE + mt * 16, d[mt][1]);
        atomicAdd(o + mt * 16 + 8, d[mt][2]);
        atomicAdd(o + X16_ASTRIDE + mt * 16 + 8, d[mt][3]);
    }
}

template <int MT, int... RT>
__device__ __forceinline__ void x16_tiles(const uint32_t (&w)[12], const uint4 (&xa)[MT][4][2], uint32_t tbl, float* __restrict__ sa, int g, int t,
                                          std::integer_sequence<int, RT...>) {
    (x16_tile<MT, RT>(w, xa, tbl, sa, g, t), ...);
}

template <int MT>
__global__ void __launch_bounds__(X16_WARPS * 32, 2)
k_gemv_x16(cbl_x16 m, const __half* __restrict__ xp, int B, int Bpad, int Cpad, void* __restrict__ y, int ydtype, int64_t ldy,
           float* __restrict__ acc_g, unsigned int* __restrict__ counters, int Rpad, int PR, int KS) {
    extern __shared__ __align__(16) unsigned char x16_smem[];
    uint4* s_table = (uint4*)x16_smem;
    float* s_acc = (float*)(x16_smem + 65536);
    __shared__ unsigned int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int pr = blockIdx.x % PR, ks = blockIdx.x / PR;
    const int rb_lo = (int)((int64_t)pr * m.nrb / PR), rb_hi = (int)((int64_t)(pr + 1) * m.nrb / PR);
    const int KB = (m.nkr + X16_WARPS - 1) / X16_WARPS;
    const int kb_lo = (int)((int64_t)ks * KB / KS), kb_hi = (int)((int64_t)(ks + 1) * KB / KS);
    const uint32_t tbl = cbl_smem_u32(s_table);
    const uint4* words = (const uint4*)m.words;
    const float* xinv = (const float*)(xp + (int64_t)Bpad * Cpad);
    bool waited = false;

    for (int rb0 = rb_lo; rb0 < rb_hi; rb0 += X16_NR) {
        const int nr = min(X16_NR, rb_hi - rb0);
        for (int i = tid; i < nr * X16_ATILE; i += X16_WARPS * 32) s_acc[i] = 0.f;
        for (int book = 0; book < m.books; book++) {
            __syncthreads();                                   // previous readers of the table, the zeroed sums
            const uint4* tb = (const uint4*)(book ? m.table2 : m.table);
            for (int i = tid; i < 4096; i += X16_WARPS * 32) s_table[i] = __ldg(tb + i);
            if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            __syncthreads();
            for (int kb = kb_lo; kb < kb_hi; kb++) {
                const int kr = kb * X16_WARPS + warp;
                if (kr >= m.nkr) continue;
                uint4 xa[MT][4][2];
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int tok = mt * 16 + h * 8 + g;
                        const uint4* xr = (const uint4*)(xp + (int64_t)tok * Cpad) + kr * 16 + t;
#pragma unroll
                        for (int j = 0; j < 4; j++) xa[mt][j][h] = tok < Bpad ? __ldg(xr + 4 * j) : make_uint4(0, 0, 0, 0);
                    }
                const uint4* wp = words + (((int64_t)book * m.nkr + kr) * m.nrb + rb0) * 96 + lane;
                // warps start at different row blocks so that their additions land in different sums
                int ri = warp % nr;
                uint32_t w[12];
                {
                    const uint4* p = wp + (int64_t)ri * 96;
#pragma unroll
                    for (int q = 0; q < 3; q++) { uint4 v = cbl_ldg_stream(p + 32 * q); w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w; }
                }
                for (int it = 0; it < nr; it++) {
                    const int rn = ri + 1 == nr ? 0 : ri + 1;
                    uint32_t wn[12];
                    if (it + 1 < nr) {
                        const uint4* p = wp + (int64_t)rn * 96;
#pragma unroll
                        for (int q = 0; q < 3; q++) { uint4 v = cbl_ldg_stream(p + 32 * q); wn[4 * q] = v.x; wn[4 * q + 1] = v.y; wn[4 * q + 2] = v.z; wn[4 * q + 3] = v.w; }
                    }
                    x16_tiles<MT>(w, xa, tbl, s_acc + ri * X16_ATILE, g, t, std::make_integer_sequence<int, 8>{});
                    if (it + 1 < nr) {
#pragma unroll
                        for (int k = 0; k < 12; k++) w[k] = wn[k];
                    }
                    ri = rn;
                }
            }
        }
        if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
        __syncthreads();
        const int row = tid & 63, tq = tid >> 6;
        if (KS == 1) {
            for (int i = 0; i < nr; i++) {
                const int r = (rb0 + i) * 64 + row;
                if (r >= m.R) continue;
                const float rs = __half2float(((const __half*)m.row_scale)[r]);
#pragma unroll
                for (int q = 0; q < 16 * MT / X16_TQ; q++) {
                    const int tok = tq + X16_TQ * q;
                    if (tok < B) cbl_store_out(y, ydtype, (int64_t)tok * ldy + r, s_acc[i * X16_ATILE + row * X16_ASTRIDE + tok] * xinv[tok] * rs);
                }
            }
        } else {
            for (int i = 0; i < nr; i++) {
                const int r = (rb0 + i) * 64 + row;
#pragma unroll
                for (int q = 0; q < 16 * MT / X16_TQ; q++) {
                    const int tok = tq + X16_TQ * q;
                    if (tok < B) atomicAdd(acc_g + (int64_t)tok * Rpad + r, s_acc[i * X16_ATILE + row * X16_ASTRIDE + tok]);
                }
            }
            __threadfence();
            __syncthreads();
            for (int i = 0; i < nr; i++) {
                if (tid == 0) s_last = atomicAdd(counters + rb0 + i, 1u) == (unsigned)(KS - 1);
                __syncthreads();
                const bool last = s_last != 0;
                __syncthreads();
                if (!last) continue;
                __threadfence();
                const int r = (rb0 + i) * 64 + row;
                const float rs = r < m.R ? __half2float(((const __half*)m.row_scale)[r]) : 0.f;
#pragma unroll
                for (int q = 0; q < 16 * MT / X16_TQ; q++) {
                    const int tok = tq + X16_TQ * q;
                    if (tok < B) {
                        float* a = acc_g + (int64_t)tok * Rpad + r;
                        const float v = __ldcg(a);
                        *a = 0.f;
                        if (r < m.R) cbl_store_out(y, ydtype, (int64_t)tok * ldy + r, v * xinv[tok] * rs);
                    }
                }
                if (tid == 0) counters[rb0 + i] = 0;
            }
        }
        __syncthreads();
    }
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
}

extern "C" size_t cbl_gemv_x16_workspace_bytes(int32_t R) {
    if (R <= 0) return 16;
    size_t nrb = ((size_t)R + 63) / 64;
    return 32 * nrb * 64 * 4 + nrb * 4;
}

// Row parts x column splits of a launch: the fewest block iterations on the longest block, the fewest splits among equals.
static void x16_shape(int nrb, int KB, int sms, int& PR, int& KS) {
    long best = -1;
    PR = 1; KS = 1;
    for (int ks = 1; ks <= KB && ks <= sms; ks++) {
        int pr = sms / ks;
        if (pr > nrb) pr = nrb;
        if (pr < 1) pr = 1;
        long cost = (long)cbl_ceil_div(nrb, pr) * cbl_ceil_div(KB, ks);
        if (best < 0 || cost < best) { best = cost; PR = pr; KS = ks; }
    }
}

template <int MT>
static int launch_x16(const cbl_x16* m, const void* xp, int B, void* y, int ydtype, int64_t ldy, void* workspace, cudaStream_t st) {
    const size_t smem = 65536 + (size_t)X16_NR * X16_ATILE * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemv_x16<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    int PR, KS;
    x16_shape(m->nrb, cbl_ceil_div(m->nkr, X16_WARPS), 2 * cbl_sm_count(), PR, KS);   // two blocks per SM
    const int Bpad = (B + 7) / 8 * 8, Cpad = (m->C + 511) / 512 * 512, Rpad = m->nrb * 64;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(PR * KS);
    cfg.blockDim = dim3(X16_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    float* acc = (float*)workspace;
    unsigned int* counters = (unsigned int*)(acc + (size_t)32 * Rpad);
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_x16<MT>, *m, (const __half*)xp, B, Bpad, Cpad, y, ydtype, ldy, acc, counters, Rpad, PR, KS));
    return cbl_check_launch();
}

extern "C" int cbl_gemv_x16(const cbl_x16* m, const void* xp, int32_t B, void* y, int ydtype, int64_t ldy, void* workspace, cbl_stream s) {
    if (!m || !m->words || !m->table || !m->row_scale || !xp || !y || !workspace) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->table2) return CBL_EINVAL;
    if (B < 1 || ldy < m->R || m->C % 8 || m->nkr != cbl_ceil_div(m->C / 8, 16) || m->nrb != cbl_ceil_div(m->R, 64)) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (B > 32) return CBL_EUNSUPPORTED;
    if (((uintptr_t)m->words % 16) || ((uintptr_t)m->table % 16) || ((uintptr_t)xp % 16) || ((uintptr_t)workspace % 16)) return CBL_EINVAL;
    if (m->R == 0) return CBL_OK;
    if (B <= 16) return launch_x16<1>(m, xp, B, y, ydtype, ldy, workspace, (cudaStream_t)s);
    return launch_x16<2>(m, xp, B, y, ydtype, ldy, workspace, (cudaStream_t)s);
}

// ------------------------------------------------------------------------------------ l8 product
//
// Work decomposition: the (tile, row group) pairs of a matrix, tile-major, are cut into gridDim.x equal
// contiguous ranges (a row group = 4 rows).  A thread block walks its range NT groups at a time; the
// groups' tag words are staged by bulk copies (cp.async.bulk + mbarrier) into a ring of shared-memory
// stages that runs L8_STAGES iterations ahead, across tile boundaries and across the table builds.
constexpr int L8_COL_WORDS = 4096 + 4;    // column stride of the table in words: the pad keeps the build's stores conflict-free
constexpr int L8_RING_BYTES = 73728;      // 3 planes x 16 bytes x (NT * stages) groups
constexpr uint32_t L8_WAIT_LIMIT = 1u << 20;   // mbarrier polls before a wait gives up

extern "C" size_t cbl_gemv_l8_workspace_bytes(int32_t R) {
    if (R < 0) return 0;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    return Rpad * 4 + 16;
}

__device__ __forceinline__ float l8_row_sum(uint32_t a, uint32_t b, uint32_t c, uint32_t lut) {
    // 8 tags of 12 bits in the 96-bit stream (a, b, c); byte offset = tag * 4 inside each column's table
    float s0 = cbl_lds_f32(lut + 0 * L8_COL_WORDS * 4 + ((a << 2) & 0x3FFCu));
    float s1 = cbl_lds_f32(lut + 1 * L8_COL_WORDS * 4 + ((a >> 10) & 0x3FFCu));
    float s2 = cbl_lds_f32(lut + 2 * L8_COL_WORDS * 4 + (__funnelshift_r(a, b, 22) & 0x3FFCu));
    float s3 = cbl_lds_f32(lut + 3 * L8_COL_WORDS * 4 + ((b >> 2) & 0x3FFCu));
    float s4 = cbl_lds_f32(lut + 4 * L8_COL_WORDS * 4 + ((b >> 14) & 0x3FFCu));
    float s5 = cbl_lds_f32(lut + 5 * L8_COL_WORDS * 4 + (__funnelshift_r(b, c, 26) & 0x3FFCu));
    float s6 = cbl_lds_f32(lut + 6 * L8_COL_WORDS * 4 + ((c >> 6) & 0x3FFCu));
    float s7 = cbl_lds_f32(lut + 7 * L8_COL_WORDS * 4 + ((c >> 18) & 0x3FFCu));
    return ((s0 + s1) + (s2 + s3)) + ((s4 + s5) + (s6 + s7));
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


// Up to L8_MAX_GROUP matrices that share one activation vector (q|k|v, gate|up) run as ONE launch:
// their tiles form one list, the work split and the tag ring run across matrix boundaries.
constexpr int L8_MAX_GROUP = 4;
struct L8Launch {
    int n;                         // matrices in the group
    int tile0[L8_MAX_GROUP + 1];   // prefix sums of their tile counts
    cbl_l8 m[L8_MAX_GROUP];
    float* acc[L8_MAX_GROUP];      // fp32 row accumulators of each matrix (zero on entry)
    void* y[L8_MAX_GROUP];
    const uint32_t* calls;         // optional: completed-call counter; call e = *calls + 1 accumulates into
    int64_t acc_stride;            // acc[0] + (e & 1) * acc_stride (two alternating buffers, see cbl_gemv_l8_ar)
};

// Work split.  The (tile, row group) pairs of the launch, tile-major over all its matrices, are cut into one
// contiguous range per block: first tile + first group, last tile + end group, whole tiles in between.
// The host plans the cut so that the SLOWEST block is as fast as possible under a simple cost model - a table
// build costs about 0.8 lookup iterations, an iteration covers up to NT row groups of one tile - and passes
// the ranges as a kernel parameter (blocks beyond the plan's count exit at once).
constexpr int L8_MAX_BLOCKS = 160;
struct L8Plan {
    int nblocks;
    int4 r[L8_MAX_BLOCKS];          // {tile_first, g_first, tile_last, g_end}
};

__host__ __device__ inline int l8_matrix_of(const L8Launch& P, int tl) {
    int mi = 0;
    while (mi + 1 < P.n && tl >= P.tile0[mi + 1]) mi++;
    return mi;
}

// Greedy sweep: blocks take work in order, each up to a cost budget T.  Returns the number of blocks used
// (and fills `out` if given); more than `maxb` means T is too small.
static int l8_sweep(const L8Launch& P, int NT, double T, int maxb, L8Plan* out) {
    const double B = 0.8;
    const int ntile = P.tile0[P.n];
    int nb = 0, t = 0, g = 0;
    while (t < ntile) {
        if (nb >= maxb) return maxb + 1;
        double c = 0.0;
        int4 r = make_int4(t, g, t, g);
        while (t < ntile) {
            const int ng = P.m[l8_matrix_of(P, t)].Rpad >> 2;
            const int k = (int)(T - c - B + 1e-9);              // whole iterations that still fit
            if (k < 1) {
                if (c == 0.0) return maxb + 1;                     // even an empty block cannot afford one tile
                break;
            }
            const int rem = ng - g;
            const int take = rem < k * NT ? rem : k * NT;
            c += B + (double)((take + NT - 1) / NT);
            r.z = t;
            r.w = g + take;
            g += take;
            if (g == ng) { t++; g = 0; } else break;
        }
        if (out) out->r[nb] = r;
        nb++;
    }
    if (out) out->nblocks = nb;
    return nb;
}

static void l8_make_plan(const L8Launch& P, int NT, int maxb, L8Plan* plan) {
    double lo = 1.8, hi = 1.8;
    for (int t = 0; t < P.tile0[P.n]; t++) hi += 0.8 + (double)(((P.m[l8_matrix_of(P, t)].Rpad >> 2) + NT - 1) / NT);
    for (int it = 0; it < 40 && hi - lo > 0.01; it++) {
        const double mid = 0.5 * (lo + hi);
        if (l8_sweep(P, NT, mid, maxb, nullptr) <= maxb) hi = mid; else lo = mid;
    }
    l8_sweep(P, NT, hi, maxb, plan);
}

template <int NT>
__global__ void __launch_bounds__(NT, 1) k_gemv_l8(const __grid_constant__ L8Launch P, const __grid_constant__ L8Plan plan,
                                                   const void* __restrict__ x, int xdtype, unsigned int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int STAGES = L8_RING_BYTES / (NT * 48);
    constexpr int NWARP = NT / 32, NIT = 256 / NWARP;
    float* s_lut = (float*)smem;                                   // [8][L8_COL_WORDS]
    unsigned char* s_ring = smem + 8 * L8_COL_WORDS * 4;           // [STAGES][3][NT] uint4
    __shared__ __align__(8) unsigned long long s_bar[2 * STAGES];  // full[STAGES] (tags landed), empty[STAGES] (every warp has read them)
    __shared__ uint32_t s_b0[32];                                  // B fragment of the tile's activations, per lane
    __shared__ float s_inv;
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    if ((int)blockIdx.x >= plan.nblocks) return;
    const int4 rg = plan.r[blockIdx.x];
    const int tile_first = rg.x, tile_last = rg.z;
    if (tile_last < tile_first) return;
    CBL_MARK(0);
    // Programmatic dependent launch: let the next kernel in the stream (the finish kernel) get resident now;
    // this kernel itself waits for its predecessor only where it first touches data that depends on it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    auto matrix_of = [&](int tl) { return l8_matrix_of(P, tl); };
    // row groups [lo, hi) of tile tl that belong to this block
    auto seg = [&](int tl, int& mi, int& lo, int& hi) {
        mi = matrix_of(tl);
        lo = tl == tile_first ? rg.y : 0;
        hi = tl == tile_last ? rg.w : (P.m[mi].Rpad >> 2);
    };
    const uint32_t lut = cbl_smem_u32(s_lut), ring = cbl_smem_u32(s_ring), bar0 = cbl_smem_u32(s_bar);
    // iterations of this block: each covers up to NT row groups of one tile
    int nit = 0;
    for (int tl = tile_first; tl <= tile_last; tl++) {
        int mi, lo, hi;
        seg(tl, mi, lo, hi);
        nit += (hi - lo + NT - 1) / NT;
    }
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < STAGES; i++) {
            l8_mbar_init(bar0 + 8 * i, 3);                      // full: one arrival per tag plane
            l8_mbar_init(bar0 + 8 * (STAGES + i), NWARP);       // empty: one arrival per consuming warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Producers: lane 0 of warps 0..2 each stage one of the three tag planes; every producer keeps its
    // own cursor over the block's iterations.  Consumers: all threads.
    const bool producer = lane == 0 && warp < 3;
    int ptile = tile_first, pmi, plo, phi, pit = 0;
    seg(ptile, pmi, plo, phi);
    int pg = plo;
    auto issue = [&]() {
        const cbl_l8& mm = P.m[pmi];
        const int ng = mm.Rpad >> 2;
        const int n = min(NT, phi - pg);
        const int stage = pit % STAGES;
        const uint32_t bar = bar0 + 8 * stage, dst = ring + stage * (NT * 48) + warp * (NT * 16);
        l8_mbar_expect_tx(bar, (uint32_t)n * 16u);
        l8_bulk_g2s(dst, (const uint4*)mm.words + ((int64_t)(ptile - P.tile0[pmi]) * 3 + warp) * ng + pg, (uint32_t)n * 16u, bar);
        pg += NT;
        pit++;
        if (pg >= phi && ptile < tile_last) { ptile++; seg(ptile, pmi, plo, phi); pg = plo; }
    };
    if (producer) issue();                                 // stage 0 now; the others after the first book reads are in flight
    CBL_MARK(7);
    // Per-tile inputs of the table build: the book's A fragments (two 16-codeword blocks per lane and load)
    // and, in one warp only, the tile's 64 activations (every block reads the same few lines: keep the
    // request count low).  B fragment: k = 2t, 2t+1 of column n = g.
    constexpr int XWARP = 3;
    uint4 af[NIT / 2];
    float x0 = 0.f, x1 = 0.f;
    float* acc0 = P.acc[0];                                // may be redirected to the call's buffer (single-matrix launches)
    auto request = [&](int tl) {
        const int mi = matrix_of(tl);
        const cbl_l8& mm = P.m[mi];
        const int ntile1 = mm.ntile / mm.books, lt = tl - P.tile0[mi];
        const int book = lt / ntile1, ctile = lt - book * ntile1;
        const uint4* fr = (const uint4*)(book ? mm.frag2 : mm.frag);
        // all blocks read the same 64 KB at the same time: start each block at a different eighth of the book
#pragma unroll
        for (int i = 0; i < NIT / 2; i++) {
            const int ii = (i + (int)blockIdx.x) % (NIT / 2);
            af[i] = __ldg(fr + (warp + ii * NWARP) * 32 + lane);
        }
        if (tl == tile_first) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // x and the accumulators come from earlier kernels
            if (P.calls) acc0 += (int64_t)((__ldcg(P.calls) + 1u) & 1u) * P.acc_stride;
        }
        if (warp == XWARP) {
            const int chunk = ctile * 8 + g;
            x0 = x1 = 0.f;
            if (chunk < (mm.C >> 3)) {
                x0 = cbl_load_in(x, xdtype, (int64_t)chunk * 8 + 2 * t);
                x1 = cbl_load_in(x, xdtype, (int64_t)chunk * 8 + 2 * t + 1);
            }
        }
    };
    request(tile_first);

    int tile = tile_first, cmi, clo, chi, built = -1;
    seg(tile, cmi, clo, chi);
    int cg = clo;
    for (int it = 0; it < nit; it++) {
        if (tile != built) {
            // ---- build T[c][e] for the tile's 8 chunk columns (its fragments and activations were requested
            // before the previous tile's lookups, or before the loop for the first tile)
            if (it == 0 && producer)
                for (int i = 1; i < STAGES && i < nit; i++) issue();
            if (warp == XWARP) {
                float mx = fmaxf(fabsf(x0), fabsf(x1));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                // power-of-two pre-scale so that fp16(x * sc) neither overflows nor underflows; undone on the fp32 result
                const int k = cbl_scale_exp(mx);
                const float sc = ldexpf(1.f, -k);
                __half2 xb = __floats2half2_rn(x0 * sc, x1 * sc);
                s_b0[lane] = *(const uint32_t*)&xb;
                if (lane == 0) s_inv = ldexpf(1.f, k);
            }
            __syncthreads();                               // every reader of the previous table is done; s_b0 is published
            const uint32_t b0 = s_b0[lane];
            const float inv = s_inv;
            if (it == 0) CBL_MARK(10);
#pragma unroll
            for (int i = 0; i < NIT / 2; i++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int e0 = ((warp + ((i + (int)blockIdx.x) % (NIT / 2)) * NWARP) * 2 + h) * 16;
                    float c[4];
                    cbl_mma1688(c, h ? af[i].z : af[i].x, h ? af[i].w : af[i].y, b0);
                    float* p = s_lut + (2 * t) * L8_COL_WORDS + e0 + g;
                    p[0] = c[0] * inv;
                    p[L8_COL_WORDS] = c[1] * inv;
                    p[8] = c[2] * inv;
                    p[L8_COL_WORDS + 8] = c[3] * inv;
                }
            }
            built = tile;
            if (tile < tile_last) request(tile + 1);       // in flight during this tile's lookups
            __syncthreads();
            if (it == 0) CBL_MARK(1);
        }
        // Warps run through the stages on their own: no block-wide barrier per iteration.  A producer lane refills
        // the stage of the previous iteration once every warp has released it.  After a wait has expired the
        // loop only keeps its shape (the table builds contain block-wide barriers) and does no more work.
        bool dead = *(volatile int*)&s_abort != 0;
        const int stage = it % STAGES;
        const int n = min(NT, chi - cg);
        if (producer && it >= 1 && pit < nit && !dead) {
            if (l8_mbar_wait(bar0 + 8 * (STAGES + (it - 1) % STAGES), (uint32_t)((it - 1) / STAGES) & 1u)) issue();
            else { s_abort = 1; dead = true; }
        }
        if (!dead && !l8_mbar_wait(bar0 + 8 * stage, (uint32_t)(it / STAGES) & 1u)) { s_abort = 1; dead = true; }
        uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0, w2 = w0;
        if (!dead && tid < n) {
            const uint32_t src = ring + stage * (NT * 48) + tid * 16;
            w0 = cbl_lds128(src);
            w1 = cbl_lds128(src + NT * 16);
            w2 = cbl_lds128(src + 2 * NT * 16);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar0 + 8 * (STAGES + stage)) : "memory");
        if (it == 0) CBL_MARK(2);
        if (!dead && tid < n) {
            float r0 = l8_row_sum(w0.x, w1.x, w2.x, lut);
            float r1 = l8_row_sum(w0.y, w1.y, w2.y, lut);
            float r2 = l8_row_sum(w0.z, w1.z, w2.z, lut);
            float r3 = l8_row_sum(w0.w, w1.w, w2.w, lut);
            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"((cmi ? P.acc[cmi] : acc0) + 4 * (int64_t)(cg + tid)), "f"(r0), "f"(r1),
                         "f"(r2), "f"(r3)
                         : "memory");
        }
        cg += NT;
        if (cg >= chi && tile < tile_last) { tile++; seg(tile, cmi, clo, chi); cg = clo; }
    }
    __syncthreads();
    if (s_abort) {
        // a staged copy never completed: report, give the copies still in flight a bounded time, leave
        if (tid == 0) {
            atomicExch(status, 1u);
            for (int i = 0; i < STAGES; i++) (void)l8_mbar_wait(bar0 + 8 * i, 0u);
        }
        return;
    }
    CBL_MARK(3);
}

// y[r] = round(row_scale[r] * acc[r]); acc[r] = 0.  Four rows per thread; blockIdx.y = matrix of the group.
__global__ void __launch_bounds__(256) k_l8_finish(const __grid_constant__ L8Launch P, int ydtype) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");          // every partial sum of the product kernel has landed
    const int mi = blockIdx.y;
    const cbl_l8& mm = P.m[mi];
    const int gi = blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= (mm.Rpad >> 2)) return;
    float4* acc = (float4*)P.acc[mi];
    const float4 v = __ldcg(acc + gi);
    __stcg(acc + gi, make_float4(0.f, 0.f, 0.f, 0.f));
    const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int r = gi * 4 + u;
        if (r < mm.R) cbl_store_out(P.y[mi], ydtype, r, vv[u] * __half2float(((const __half*)mm.row_scale)[r]));
    }
}

// Book in mma.m16n8k8 A-fragment order: uint4 [128][32] = {a0, a1 of codeword block 2p, a0, a1 of block 2p+1}
// for lane (g, t): a0 = codeword (16*blk + g) values 2t, 2t+1; a1 = codeword (16*blk + g + 8) values 2t, 2t+1.
__global__ void __launch_bounds__(256) k_repack_book(const uint32_t* __restrict__ table, uint4* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;       // 0 .. 4095
    const int lane = i & 31, p = i >> 5, g = lane >> 2, t = lane & 3;
    uint4 v;
    v.x = table[((2 * p) * 16 + g) * 4 + t];
    v.y = table[((2 * p) * 16 + g + 8) * 4 + t];
    v.z = table[((2 * p + 1) * 16 + g) * 4 + t];
    v.w = table[((2 * p + 1) * 16 + g + 8) * 4 + t];
    out[i] = v;
}

extern "C" size_t cbl_book_frag_bytes(void) { return 65536; }

extern "C" int cbl_repack_book(const void* table, void* out, cbl_stream s) {
    if (!table || !out || ((uintptr_t)table % 4) || ((uintptr_t)out % 16)) return CBL_EINVAL;
    k_repack_book<<<16, 256, 0, (cudaStream_t)s>>>((const uint32_t*)table, (uint4*)out);
    return cbl_check_launch();
}

static int l8_threads() {
    static int v = 0;
    if (!v) {
        const char* e = getenv("CBL_L8_THREADS");
        v = e ? atoi(e) : 512;
        if (v != 256 && v != 512) v = 512;
    }
    return v;
}

static int check_l8(const cbl_l8* m) {
    if (!m || !m->words || !m->frag || !m->row_scale) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->frag2) return CBL_EINVAL;
    if (m->R < 0 || m->C <= 0 || m->C % 8 || m->Rpad != (m->R + 3) / 4 * 4) return CBL_EINVAL;
    if (m->ntile != m->books * cbl_ceil_div(m->C / 8, 8)) return CBL_EINVAL;
    if (((uintptr_t)m->words % 16) || ((uintptr_t)m->frag % 16)) return CBL_EINVAL;
    if (m->books == 2 && ((uintptr_t)m->frag2 % 16)) return CBL_EINVAL;
    return CBL_OK;
}

template <int NT>
static int launch_l8(const L8Launch& P, const void* x, int xdtype, int ydtype, unsigned int* status, cudaStream_t st, bool finish = true) {
    const size_t smem = (size_t)8 * L8_COL_WORDS * 4 + L8_RING_BYTES;
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemv_l8<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    // one block per SM at most; a tile is cut into row ranges of at least 128 groups (512 rows) each
    int ntile = P.tile0[P.n], max_groups = 0, min_groups = 1 << 30;
    for (int i = 0; i < P.n; i++) {
        max_groups = max_groups > (P.m[i].Rpad >> 2) ? max_groups : (P.m[i].Rpad >> 2);
        min_groups = min_groups < (P.m[i].Rpad >> 2) ? min_groups : (P.m[i].Rpad >> 2);
    }
    int grid = cbl_sm_count();
    int parts = min_groups / 128;
    if (parts < 1) parts = 1;
    if ((int64_t)ntile * parts < grid) grid = ntile * parts;
    if (grid > L8_MAX_BLOCKS) grid = L8_MAX_BLOCKS;
    // plan cache: the cut depends only on the shapes of the group
    static std::mutex mu;
    static std::map<std::vector<int>, L8Plan> cache;
    std::vector<int> key = {NT, grid, P.n};
    for (int i = 0; i < P.n; i++) { key.push_back(P.m[i].ntile); key.push_back(P.m[i].Rpad); }
    L8Plan plan;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it == cache.end()) {
            l8_make_plan(P, NT, grid, &plan);
            cache.emplace(key, plan);
        } else plan = it->second;
    }
    const L8Launch& Q = P;
    static int pdl = -1;
    if (pdl < 0) { const char* e = getenv("CBL_PDL"); pdl = (e && atoi(e) == 0) ? 0 : 1; }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_gemv_l8<NT>, Q, plan, x, xdtype, status));
    if (!finish) return cbl_check_launch();
    cfg.gridDim = dim3(cbl_ceil_div(max_groups, 256), P.n);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_l8_finish, P, ydtype));
    return cbl_check_launch();
}

// Fills the launch descriptor of a group: accumulators carved from `workspace` in order, the status word after them.
static int l8_group(const cbl_l8* mats, int32_t n, const void* x, int xdtype, void* const* ys, void* workspace, L8Launch& P,
                    unsigned int*& status) {
    if (!mats || !x || !workspace || n < 1) return CBL_EINVAL;
    if (n > L8_MAX_GROUP) return CBL_EUNSUPPORTED;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if ((uintptr_t)workspace % 16) return CBL_EINVAL;
    P.n = 0;
    P.tile0[0] = 0;
    size_t off = 0;
    for (int i = 0; i < n; i++) {
        int rc = check_l8(mats + i);
        if (rc) return rc;
        if (mats[i].C != mats[0].C) return CBL_EINVAL;          // one shared activation vector
        if (ys && !ys[i]) return CBL_EINVAL;
        if (mats[i].R == 0) continue;
        P.m[P.n] = mats[i];
        P.acc[P.n] = (float*)((char*)workspace + off);
        P.y[P.n] = ys ? ys[i] : nullptr;
        P.tile0[P.n + 1] = P.tile0[P.n] + mats[i].ntile;
        off += (size_t)mats[i].Rpad * 4;
        P.n++;
    }
    P.calls = nullptr;
    P.acc_stride = 0;
    status = (unsigned int*)((char*)workspace + off);
    return CBL_OK;
}

static int l8_launch_any(const L8Launch& P, const void* x, int xdtype, int ydtype, unsigned int* status, cudaStream_t st, bool finish) {
    if (l8_threads() == 256) return launch_l8<256>(P, x, xdtype, ydtype, status, st, finish);
    return launch_l8<512>(P, x, xdtype, ydtype, status, st, finish);
}

extern "C" int cbl_gemv_l8_multi(const cbl_l8* mats, int32_t n, const void* x, int xdtype, void* const* ys, int ydtype,
                                 void* workspace, cbl_stream s) {
    if (!ys) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    L8Launch P;
    unsigned int* status = nullptr;
    int rc = l8_group(mats, n, x, xdtype, ys, workspace, P, status);
    if (rc) return rc;
    if (P.n == 0) return CBL_OK;
    return l8_launch_any(P, x, xdtype, ydtype, status, (cudaStream_t)s, true);
}

extern "C" int cbl_gemv_l8(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* workspace, cbl_stream s) {
    if (!m || !y) return CBL_EINVAL;
    void* ys[1] = {y};
    return cbl_gemv_l8_multi(m, 1, x, xdtype, ys, ydtype, workspace, s);
}

// Reads the status word a product leaves in its work space (0 = ok, nonzero = a bounded device-side
// wait expired and the output is invalid).  Synchronises the stream.
extern "C" int cbl_gemv_l8_status(const void* workspace, int32_t R, cbl_stream s) {
    if (!workspace || R < 0) return CBL_EINVAL;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    unsigned int v = 0;
    CBL_CUDA(cudaMemcpyAsync(&v, (const char*)workspace + Rpad * 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    CBL_CUDA(cudaStreamSynchronize((cudaStream_t)s));
    return v ? CBL_ETIMEOUT : CBL_OK;
}

// ------------------------------------------------------------------------------------ batch-1 products with a decode-step epilogue
//
// In a decode step most products are followed by a small operator on their output vector.  These entry
// points run that operator inside the finish kernel (one launch less per product, no round trip of the
// vector through memory); results are identical to the separate operators of the step library because
// the product is rounded to the model's 16-bit type first, exactly as if it had been stored.
//   gate|up  -> silu(gate) * up                      (cbl_silu_mul)
//   o / down -> residual add + RMSNorm               (cbl_add_rmsnorm): the finish kernel's blocks form one
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
    if (gi >= (mg.Rpad >> 2)) return;
    float4* ag = (float4*)P.acc[0];
    float4* au = (float4*)P.acc[1];
    const float4 g = __ldcg(ag + gi), u = __ldcg(au + gi);
    __stcg(ag + gi, make_float4(0.f, 0.f, 0.f, 0.f));
    __stcg(au + gi, make_float4(0.f, 0.f, 0.f, 0.f));
    const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int r = gi * 4 + k;
        if (r < mg.R) {
            const float a = l8_f(cbl_cvt_out<T>(gv[k] * __half2float(((const __half*)mg.row_scale)[r])));
            const float b = l8_f(cbl_cvt_out<T>(uv[k] * __half2float(((const __half*)mu.row_scale)[r])));
            const float sl = l8_f(cbl_cvt_out<T>(a / (1.f + __expf(-a))));
            out[r] = cbl_cvt_out<T>(sl * b);
        }
    }
}

constexpr int L8_NORM_MAX_CTAS = 8;          // portable cluster size: up to 8 x 1024 rows
template <typename T>
__global__ void __launch_bounds__(256) k_l8_finish_addnorm(const __grid_constant__ L8Launch P, float* __restrict__ h, const T* __restrict__ w,
                                                           float eps, T* __restrict__ xout) {
    l8_pdl_enter();
    __shared__ float s_warp[8];
    __shared__ float s_ss, s_tot;
    const cbl_l8& mm = P.m[0];
    const int tid = threadIdx.x, gi = blockIdx.x * blockDim.x + tid, nb = gridDim.x;
    float hv[4] = {0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
    if (gi < (mm.Rpad >> 2)) {
        float4* acc = (float4*)P.acc[0];
        const float4 v = __ldcg(acc + gi);
        __stcg(acc + gi, make_float4(0.f, 0.f, 0.f, 0.f));
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int r = gi * 4 + k;
            if (r < mm.R) {
                hv[k] = h[r] + l8_f(cbl_cvt_out<T>(vv[k] * __half2float(((const __half*)mm.row_scale)[r])));
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
    if (gi < (mm.Rpad >> 2)) {
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
    // one output element of matrix mi: take the sum, clear it, scale, round, add the bias in the 16-bit type
    auto take = [&](int mi, int r, int bcol) {
        float* a = P.acc[mi] + r;
        const float v = __ldcg(a);
        __stcg(a, 0.f);
        const float y = l8_f(cbl_cvt_out<T>(v * __half2float(((const __half*)P.m[mi].row_scale)[r])));
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

extern "C" int cbl_gemv_l8_silu_mul(const cbl_l8* gate_up, const void* x, int xdtype, void* out, int dtype, void* workspace, cbl_stream s) {
    if (!out || (dtype != CBL_F16 && dtype != CBL_BF16)) return CBL_EINVAL;
    L8Launch P;
    unsigned int* status = nullptr;
    int rc = l8_group(gate_up, 2, x, xdtype, nullptr, workspace, P, status);
    if (rc) return rc;
    if (gate_up[0].R != gate_up[1].R) return CBL_EINVAL;
    if (P.n == 0) return CBL_OK;
    const cudaStream_t st = (cudaStream_t)s;
    rc = l8_launch_any(P, x, xdtype, dtype, status, st, false);
    if (rc) return rc;
    const dim3 grid(cbl_ceil_div(P.m[0].Rpad >> 2, 256));
    if (dtype == CBL_F16) return l8_finish_launch(k_l8_finish_silu<__half>, grid, dim3(256), 1, st, P, (__half*)out);
    return l8_finish_launch(k_l8_finish_silu<__nv_bfloat16>, grid, dim3(256), 1, st, P, (__nv_bfloat16*)out);
}

extern "C" int32_t cbl_gemv_l8_add_norm_max_rows(void) { return L8_NORM_MAX_CTAS * 1024; }

extern "C" int cbl_gemv_l8_add_norm(const cbl_l8* m, const void* x, int xdtype, float* h, const void* w, float eps, void* xout, int dtype,
                                    void* workspace, cbl_stream s) {
    if (!h || !w || !xout || (dtype != CBL_F16 && dtype != CBL_BF16)) return CBL_EINVAL;
    L8Launch P;
    unsigned int* status = nullptr;
    int rc = l8_group(m, 1, x, xdtype, nullptr, workspace, P, status);
    if (rc) return rc;
    if (m->R < 1) return CBL_EINVAL;
    if (m->R > L8_NORM_MAX_CTAS * 1024) return CBL_EUNSUPPORTED;
    const cudaStream_t st = (cudaStream_t)s;
    rc = l8_launch_any(P, x, xdtype, dtype, status, st, false);
    if (rc) return rc;
    const int nb = cbl_ceil_div(P.m[0].Rpad >> 2, 256);
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
    unsigned int* status = nullptr;
    int rc = l8_group(qkv, 3, x, xdtype, nullptr, workspace, P, status);
    if (rc) return rc;
    if (qkv[0].R != NH * HD || qkv[1].R != NKV * HD || qkv[2].R != NKV * HD) return CBL_EINVAL;
    const cudaStream_t st = (cudaStream_t)s;
    rc = l8_launch_any(P, x, xdtype, dtype, status, st, false);
    if (rc) return rc;
    const dim3 grid(NH + NKV);
    if (dtype == CBL_F16)
        return l8_finish_launch(k_l8_finish_rope<__half>, grid, dim3(64), 1, st, P, (const __half*)bias, pos, (int)NH, (int)NKV, (int)HD, theta,
                                (int)max_len, (__half*)q_out, (__half*)kc, (__half*)vc);
    return l8_finish_launch(k_l8_finish_rope<__nv_bfloat16>, grid, dim3(64), 1, st, P, (const __nv_bfloat16*)bias, pos, (int)NH, (int)NKV, (int)HD,
                            theta, (int)max_len, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc);
}

// ------------------------------------------------------------------------------------ row-split product + all-reduce over peer memory
//
// Tensor-parallel o / down projections: every rank multiplies its chunk range into its own fp32
// accumulators (the kernel above), then ONE kernel per rank finishes the job across GPUs without a
// collective library: it publishes "my partial sums of call e are complete" to every peer (a word
// stored into the peer's flag array over NVLink), waits - bounded - for the same word from every
// peer, reads all ranks' partial sums with plain peer loads, adds them in rank order (so every rank
// gets bit-identical results), applies the row scale and writes y.  Two accumulator buffers alternate
// by call so that a rank never overwrites sums a peer may still be reading.  The call number e lives
// in the work space and is advanced by the kernel itself, so a captured CUDA graph can be replayed.
//
// Work space of each rank (the same layout everywhere, allocated as symmetric memory by the caller,
// zero before the first call): acc[0] | acc[1] (Rpad fp32 each) | flags (uint32 per rank) | status |
// completed calls | block ticket.
constexpr int L8_AR_MAX_RANKS = 8;
constexpr uint32_t L8_AR_SPIN_LIMIT = 1u << 22;      // polls of a peer's flag before giving up (~1 s)

struct L8AllReduce {
    int rank, world, R, Rpad, ydtype;
    int64_t acc_stride;                       // floats between the two accumulator buffers
    const float* acc[L8_AR_MAX_RANKS];        // every rank's accumulator buffer 0 (peer pointers)
    uint32_t* flags[L8_AR_MAX_RANKS];         // every rank's flag array
    uint32_t* ctl;                            // this rank's {status, completed calls, ticket}
    const __half* row_scale;
    void* y;
};

extern "C" size_t cbl_gemv_l8_ar_workspace_bytes(int32_t R) {
    if (R < 0) return 0;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    return 2 * Rpad * 4 + L8_AR_MAX_RANKS * 4 + 32;
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
        if (blockIdx.x == 0) {
            __threadfence_system();
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(A.flags[tid] + A.rank), "r"(epoch) : "memory");
        }
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
    } else if (gi < (A.Rpad >> 2)) {
        const int64_t cur = (int64_t)(epoch & 1u) * A.acc_stride, nxt = (int64_t)((epoch + 1u) & 1u) * A.acc_stride;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < A.world; r++) {
            const float4 v = __ldcg((const float4*)(A.acc[r] + cur) + gi);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        __stcg((float4*)(const_cast<float*>(A.acc[A.rank]) + nxt) + gi, make_float4(0.f, 0.f, 0.f, 0.f));
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
    int rc = check_l8(m);
    if (rc) return rc;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    for (int r = 0; r < world; r++)
        if (!peer_ws[r] || ((uintptr_t)peer_ws[r] % 16)) return CBL_EINVAL;
    if (m->R == 0) return CBL_OK;
    const size_t accb = (size_t)m->Rpad * 4;
    uint32_t* ctl = (uint32_t*)((char*)peer_ws[rank] + 2 * accb + L8_AR_MAX_RANKS * 4);
    L8Launch P;
    P.n = 1;
    P.tile0[0] = 0;
    P.tile0[1] = m->ntile;
    P.m[0] = *m;
    P.acc[0] = (float*)peer_ws[rank];
    P.y[0] = y;
    P.calls = ctl + 1;
    P.acc_stride = m->Rpad;
    L8AllReduce A;
    A.rank = rank; A.world = world; A.R = m->R; A.Rpad = m->Rpad; A.ydtype = ydtype;
    A.acc_stride = m->Rpad;
    for (int r = 0; r < world; r++) {
        A.acc[r] = (const float*)peer_ws[r];
        A.flags[r] = (uint32_t*)((char*)peer_ws[r] + 2 * accb);
    }
    A.ctl = ctl;
    A.row_scale = (const __half*)m->row_scale;
    A.y = y;
    cudaStream_t st = (cudaStream_t)s;
    rc = (l8_threads() == 256) ? launch_l8<256>(P, x, xdtype, ydtype, ctl, st, false) : launch_l8<512>(P, x, xdtype, ydtype, ctl, st, false);
    if (rc) return rc;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(cbl_ceil_div(m->Rpad >> 2, 256));
    cfg.blockDim = dim3(256);
    CBL_CUDA(cudaLaunchKernelEx(&cfg, k_l8_finish_allreduce, A));
    return cbl_check_launch();
}

// Status of the last cbl_gemv_l8_ar calls on this rank's work space: CBL_ETIMEOUT if a peer's "ready" word
// did not arrive within the bounded wait (the output of that call is invalid).  Synchronises the stream
// and clears the status word.
extern "C" int cbl_gemv_l8_ar_status(void* workspace, int32_t R, cbl_stream s) {
    if (!workspace || R < 0) return CBL_EINVAL;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    char* p = (char*)workspace + 2 * Rpad * 4 + L8_AR_MAX_RANKS * 4;
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
// For them the fp32 row accumulators of the batch-1 product live in a fixed array inside the library
// image instead of a caller buffer.  The array is part of every CUDA context that loads the library
// (256 KB + 256 B per GPU, held until the process exits).
constexpr int L8_STATIC_MAX_ROWS = 65536;
static __device__ __align__(256) unsigned char g_l8_static_scratch[L8_STATIC_MAX_ROWS * 4 + 256];

extern "C" int32_t cbl_gemv_l8_static_max_rows(void) { return L8_STATIC_MAX_ROWS; }

extern "C" int cbl_gemv_l8_static(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, cbl_stream s) {
    if (!m) return CBL_EINVAL;
    if (m->R > L8_STATIC_MAX_ROWS) return CBL_EUNSUPPORTED;      // the built-in scratch holds 65536 rows at most
    // The array's name is only a host-side handle; the device address comes from the runtime, once per
    // device, with that device current.  (This first call per device should happen outside stream capture.)
    static void* scratch_addr[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return CBL_EUNSUPPORTED;
    if (!scratch_addr[dev]) {
        void* p = nullptr;
        CBL_CUDA(cudaGetSymbolAddress(&p, g_l8_static_scratch));
        scratch_addr[dev] = p;
    }
    // Every call shares the array and finds whatever the previous call left: clear the part this
    // call accumulates into (accumulators and status word) on the caller's stream first.
    const size_t bytes = cbl_gemv_l8_workspace_bytes(m->R);
    CBL_CUDA(cudaMemsetAsync(scratch_addr[dev], 0, bytes, (cudaStream_t)s));
    return cbl_gemv_l8(m, x, xdtype, y, ydtype, scratch_addr[dev], s);
}
