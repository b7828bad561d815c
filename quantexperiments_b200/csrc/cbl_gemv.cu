// Decode-time products straight from the packed tags (d = 8, 12-bit tags, 4096-entry fp16 books).
//
//   cbl_gemv_t16: batch <= 64.  The 64 KB book (128 KB for two summed books) lives in shared memory;
//                 a 16-byte codeword read lands directly in an mma.sync A fragment, the activations
//                 are the B fragment, accumulation is fp32.  Bound by shared-memory gather rate
//                 (random 16-byte reads), not by HBM.
//   cbl_gemv_x16: 9..32 tokens, one column order: activations stationary in registers.
// (The batch-1 product by activation-side tables lives in cbl_gemv1.cu.)
#include <utility>
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
        // cross-warp sum in a fixed order (deterministic), row scale, output rounding
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
            *(float4*)(s_red + ((warp * NB + nb) * 32 + lane) * 4) = make_float4(acc[0][nb][0] + acc[1][nb][0], acc[0][nb][1] + acc[1][nb][1],
                                                                                 acc[0][nb][2] + acc[1][nb][2], acc[0][nb][3] + acc[1][nb][3]);
        __syncthreads();
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
    }
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

