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
//                 finished (row scale, output rounding) by the last block to arrive per 512 rows.
#include <utility>
#include <cstdlib>
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
    k_prep_x<<<M * Bpad, 256, 0, (cudaStream_t)s>>>(x, xdtype, B, C, ldx, M > 1 ? perms : nullptr, Bpad, Cpad, (__half*)xp, xinv);
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

template <int BOOKS, int NB, int S>
__device__ __forceinline__ void t16_step(float (&acc)[NB][4], const uint32_t (&w)[BOOKS][12], uint32_t tbl,
                                         const uint4* __restrict__ xrow, int64_t xstride8) {
    // xrow points at chunk (ss*16)*4 + t of batch row g; step S adds 4 chunks
    uint4 xv[NB];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) xv[nb] = __ldg(xrow + S * 4 + nb * xstride8);
#pragma unroll
    for (int bk = 0; bk < BOOKS; bk++) {
        uint4 c0 = cbl_lds128(tbl + bk * 65536u + t16_tag_off<2 * S>(w[bk]));
        uint4 c1 = cbl_lds128(tbl + bk * 65536u + t16_tag_off<2 * S + 1>(w[bk]));
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
            cbl_mma16816(acc[nb], c0.x, c1.x, c0.y, c1.y, xv[nb].x, xv[nb].y);
            cbl_mma16816(acc[nb], c0.z, c1.z, c0.w, c1.w, xv[nb].z, xv[nb].w);
        }
    }
}

template <int BOOKS, int NB, int... S>
__device__ __forceinline__ void t16_steps(float (&acc)[NB][4], const uint32_t (&w)[BOOKS][12], uint32_t tbl,
                                          const uint4* __restrict__ xrow, int64_t xstride8, std::integer_sequence<int, S...>) {
    (t16_step<BOOKS, NB, S>(acc, w, tbl, xrow, xstride8), ...);
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
    __syncthreads();
    const uint32_t tbl = cbl_smem_u32(s_table);
    const uint4* words = (const uint4*)m.words;
    const int64_t book_stride = (int64_t)m.ntile * m.nsuper * 96;   // uint4 per book
    const int64_t xstride8 = (int64_t)8 * Cpad / 8;                 // uint4 between batch blocks of 8 rows

    for (int tile = blockIdx.x; tile < m.ntile; tile += gridDim.x) {
        const int mk = m.tile_mask ? m.tile_mask[tile] : 0;
        const float* xinv = (const float*)(xp + (int64_t)m.M * Bpad * Cpad);
        const uint4* xbase = (const uint4*)(xp + ((int64_t)mk * Bpad + g) * Cpad) + t;
        float acc[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
#pragma unroll
            for (int k = 0; k < 4; k++) acc[nb][k] = 0.f;
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
            t16_steps<BOOKS, NB>(acc, w, tbl, xbase + (int64_t)ss * 64, xstride8, std::make_integer_sequence<int, 16>{});
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
            *(float4*)(s_red + ((warp * NB + nb) * 32 + lane) * 4) = make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
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
    k_gemv_t16<BOOKS, NB><<<grid, T16_WARPS * 32, smem, st>>>(*m, (const __half*)xp, B, Bpad, Cpad, y, ydtype, ldy);
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

// ------------------------------------------------------------------------------------ l8 product
constexpr int L8_RB_ROWS = 512;           // rows per arrival block
constexpr int L8_COL_WORDS = 4096 + 4;    // column stride of the table in words: the pad keeps the build's stores conflict-free
constexpr int L8_GROUPS_PER_BLOCK = L8_RB_ROWS / 4;
constexpr int L8_MAX_WIN = 1024;          // arrival blocks one thread block can finish per segment pass

extern "C" size_t cbl_gemv_l8_workspace_bytes(int32_t R) {
    if (R < 0) return 0;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    size_t nblk = (Rpad / 4 + L8_GROUPS_PER_BLOCK - 1) / L8_GROUPS_PER_BLOCK;
    return Rpad * 4 + nblk * 4 + 16;
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

template <int NT>
__global__ void __launch_bounds__(NT, 1) k_gemv_l8(cbl_l8 m, const void* __restrict__ x, int xdtype, void* __restrict__ y,
                                                   int ydtype, float* __restrict__ acc, unsigned int* __restrict__ cnt) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* s_lut = (float*)smem;                         // [8][L8_COL_WORDS]
    __shared__ int s_win[L8_MAX_WIN];
    __shared__ int s_nwin;
    constexpr int NWARP = NT / 32, NIT = 256 / NWARP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ngroups = m.Rpad >> 2;
    const int ntile1 = m.ntile / m.books;
    const int nch = m.C >> 3;
    const int64_t total = (int64_t)m.ntile * ngroups;
    const int64_t a = total * blockIdx.x / gridDim.x, e = total * (blockIdx.x + 1) / gridDim.x;
    if (a >= e) return;
    const int tile_first = (int)(a / ngroups), tile_last = (int)((e - 1) / ngroups);
    const uint32_t lut = cbl_smem_u32(s_lut);
    if (tid == 0) s_nwin = 0;

    for (int tile = tile_first; tile <= tile_last; tile++) {
        const int g_lo = (tile == tile_first) ? (int)(a - (int64_t)tile * ngroups) : 0;
        const int g_hi = (tile == tile_last) ? (int)(e - (int64_t)tile * ngroups) : ngroups;
        // first tags of this segment: in flight while the table is built
        const uint4* wp = (const uint4*)m.words + (int64_t)tile * 3 * ngroups;
        int gi = g_lo + tid;
        uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0, w2 = w0;
        if (gi < g_hi) {
            w0 = cbl_ldg_stream(wp + gi);
            w1 = cbl_ldg_stream(wp + ngroups + gi);
            w2 = cbl_ldg_stream(wp + 2 * ngroups + gi);
        }
        // ---- build T[c][e] for the tile's 8 chunk columns
        {
            const int book = tile / ntile1, ctile = tile - book * ntile1;
            const __half* table = (const __half*)(book ? m.table2 : m.table);
            const int chunk = ctile * 8 + g;              // B fragment: k = 2t, 2t+1 of column n = g
            float x0 = 0.f, x1 = 0.f;
            if (chunk < nch) {
                x0 = cbl_load_in(x, xdtype, (int64_t)chunk * 8 + 2 * t);
                x1 = cbl_load_in(x, xdtype, (int64_t)chunk * 8 + 2 * t + 1);
            }
            float mx = fmaxf(fabsf(x0), fabsf(x1));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            // power-of-two pre-scale so that fp16(x * sc) neither overflows nor underflows; undone on the fp32 result
            const int k = cbl_scale_exp(mx);
            const float sc = ldexpf(1.f, -k), inv = ldexpf(1.f, k);
            __half2 xb = __floats2half2_rn(x0 * sc, x1 * sc);
            const uint32_t b0 = *(const uint32_t*)&xb;
            const uint32_t* tw = (const uint32_t*)table;   // 4 words per codeword
            uint32_t a0[NIT], a1[NIT];
#pragma unroll
            for (int i = 0; i < NIT; i++) {
                const int e0 = (warp + i * NWARP) * 16;
                a0[i] = __ldg(tw + (e0 + g) * 4 + t);
                a1[i] = __ldg(tw + (e0 + g + 8) * 4 + t);
            }
            __syncthreads();                               // every reader of the previous table is done
#pragma unroll
            for (int i = 0; i < NIT; i++) {
                const int e0 = (warp + i * NWARP) * 16;
                float c[4];
                cbl_mma1688(c, a0[i], a1[i], b0);
                float* p = s_lut + (2 * t) * L8_COL_WORDS + e0 + g;
                p[0] = c[0] * inv;
                p[L8_COL_WORDS] = c[1] * inv;
                p[8] = c[2] * inv;
                p[L8_COL_WORDS + 8] = c[3] * inv;
            }
            __syncthreads();
        }
        // ---- one table read per weight chunk
        while (gi < g_hi) {
            const int gn = gi + NT;
            uint4 n0 = w0, n1 = w1, n2 = w2;
            if (gn < g_hi) {
                n0 = cbl_ldg_stream(wp + gn);
                n1 = cbl_ldg_stream(wp + ngroups + gn);
                n2 = cbl_ldg_stream(wp + 2 * ngroups + gn);
            }
            float r0 = l8_row_sum(w0.x, w1.x, w2.x, lut);
            float r1 = l8_row_sum(w0.y, w1.y, w2.y, lut);
            float r2 = l8_row_sum(w0.z, w1.z, w2.z, lut);
            float r3 = l8_row_sum(w0.w, w1.w, w2.w, lut);
            asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(acc + 4 * (int64_t)gi), "f"(r0), "f"(r1), "f"(r2), "f"(r3)
                         : "memory");
            w0 = n0; w1 = n1; w2 = n2;
            gi = gn;
        }
        // ---- arrival accounting per block of 512 rows; the thread block completing a count finishes those rows
        __threadfence();
        __syncthreads();
        const int b_lo = g_lo / L8_GROUPS_PER_BLOCK, b_hi = (g_hi - 1) / L8_GROUPS_PER_BLOCK;
        for (int base = b_lo; base <= b_hi; base += L8_MAX_WIN) {
            for (int rb = base + tid; rb <= b_hi && rb < base + L8_MAX_WIN; rb += NT) {
                const int lo = max(g_lo, rb * L8_GROUPS_PER_BLOCK), hi = min(g_hi, (rb + 1) * L8_GROUPS_PER_BLOCK);
                const unsigned int n = (unsigned int)(hi - lo);
                const unsigned int expect = (unsigned int)m.ntile * (unsigned int)(min(ngroups, (rb + 1) * L8_GROUPS_PER_BLOCK) - rb * L8_GROUPS_PER_BLOCK);
                const unsigned int old = atomicAdd(cnt + rb, n);
                if (old + n == expect) s_win[atomicAdd(&s_nwin, 1)] = rb;
            }
            __syncthreads();
            const int nwin = s_nwin;
            if (nwin) {
                __threadfence();
                const int nelem = nwin * L8_RB_ROWS;
                for (int i0 = tid; i0 < nelem; i0 += 4 * NT) {
                    float v[4];
                    int row[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int i = i0 + u * NT;
                        row[u] = -1;
                        if (i < nelem) {
                            const int r = s_win[i / L8_RB_ROWS] * L8_RB_ROWS + (i % L8_RB_ROWS);
                            if (r < m.Rpad) { row[u] = r; v[u] = __ldcg(acc + r); }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (row[u] < 0) continue;
                        __stcg(acc + row[u], 0.f);
                        if (row[u] < m.R) cbl_store_out(y, ydtype, row[u], v[u] * __half2float(((const __half*)m.row_scale)[row[u]]));
                    }
                }
                for (int i = tid; i < nwin; i += NT) __stcg(cnt + s_win[i], 0u);
            }
            __syncthreads();
            if (tid == 0) s_nwin = 0;
            __syncthreads();
        }
    }
}

static int l8_threads() {
    static int v = 0;
    if (!v) {
        const char* e = getenv("CBL_L8_THREADS");
        v = e ? atoi(e) : 512;
        if (v != 256 && v != 512 && v != 1024) v = 512;
    }
    return v;
}

template <int NT>
static int launch_l8(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* workspace, cudaStream_t st) {
    const size_t smem = (size_t)8 * L8_COL_WORDS * 4;
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_gemv_l8<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    const int ngroups = m->Rpad / 4;
    int64_t total = (int64_t)m->ntile * ngroups;
    int grid = cbl_sm_count();
    // a block should own at least ~2 groups per thread, or the table build dominates
    int64_t cap = total / (2 * NT);
    if (cap < 1) cap = 1;
    if (grid > cap) grid = (int)cap;
    float* acc = (float*)workspace;
    unsigned int* cnt = (unsigned int*)((char*)workspace + (size_t)m->Rpad * 4);
    k_gemv_l8<NT><<<grid, NT, smem, st>>>(*m, x, xdtype, y, ydtype, acc, cnt);
    return cbl_check_launch();
}

extern "C" int cbl_gemv_l8(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* workspace, cbl_stream s) {
    if (!m || !m->words || !m->table || !m->row_scale || !x || !y || !workspace) return CBL_EINVAL;
    if (m->books != 1 && m->books != 2) return CBL_EINVAL;
    if (m->books == 2 && !m->table2) return CBL_EINVAL;
    if (m->R < 0 || m->C <= 0 || m->C % 8 || m->Rpad != (m->R + 3) / 4 * 4) return CBL_EINVAL;
    if (m->ntile != m->books * cbl_ceil_div(m->C / 8, 8)) return CBL_EINVAL;
    if (xdtype != CBL_F16 && xdtype != CBL_BF16 && xdtype != CBL_F32) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (((uintptr_t)m->words % 16) || ((uintptr_t)workspace % 16) || ((uintptr_t)m->table % 4)) return CBL_EINVAL;
    if (m->R == 0) return CBL_OK;
    cudaStream_t st = (cudaStream_t)s;
    switch (l8_threads()) {
        case 256: return launch_l8<256>(m, x, xdtype, y, ydtype, workspace, st);
        case 1024: return launch_l8<1024>(m, x, xdtype, y, ydtype, workspace, st);
        default: return launch_l8<512>(m, x, xdtype, y, ydtype, workspace, st);
    }
}
