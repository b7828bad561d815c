// Dense decode, tag unpacking and the load-time re-layouts (file layout -> kernel layouts).
#include <cstdlib>
#include <type_traits>
#include "cbl_common.cuh"

int g_cbl_last_cuda_error = 0;

extern "C" int cbl_version(void) { return 100; }
extern "C" int cbl_built_for_sm(void) { return 100; }
extern "C" int cbl_last_cuda_error(void) { return g_cbl_last_cuda_error; }
extern "C" const char* cbl_status_string(int status) {
    switch (status) {
        case CBL_OK: return "ok";
        case CBL_EINVAL: return "invalid argument";
        case CBL_EUNSUPPORTED: return "unsupported shape or format variant";
        case CBL_ECUDA: return "CUDA runtime error";
        case CBL_ETIMEOUT: return "bounded device-side wait expired";
        default: return "unknown status";
    }
}

int cbl_sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static int check_packed(const cbl_packed* m) {
    if (!m || !m->tags || !m->table || !m->row_scale) return CBL_EINVAL;
    if (m->R < 0 || m->C <= 0 || m->d < 1 || m->d > 16 || m->bits < 1 || m->bits > 16) return CBL_EINVAL;
    if (m->C % m->d) return CBL_EINVAL;
    if (m->G < 1 || m->M < 1 || (m->books != 1 && m->books != 2)) return CBL_EINVAL;
    if ((int64_t)m->W * 32 < (int64_t)(m->C / m->d) * m->bits) return CBL_EINVAL;
    if (m->books == 2 && (!m->tags2 || !m->table2 || m->G != 1)) return CBL_EINVAL;
    if (m->G > 1 && !m->row_book) return CBL_EINVAL;
    if (m->M > 1 && (!m->row_mask || !m->perms)) return CBL_EINVAL;
    return CBL_OK;
}

// ------------------------------------------------------------------------------------ dense decode
//
// One thread per chunk.  u = fp32(cw) [+ fp32(cw2)] rounded, then u * fp32(row_scale) rounded, then
// one rounding to the output type: the order of shapequant/packed.py:266 and masks.py:193-200.
template <typename OutT, int D, bool VEC>
__global__ void __launch_bounds__(256) k_dequant(cbl_packed m, OutT* __restrict__ out, int64_t ld, int r0, int64_t nchunks_total) {
    int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= nchunks_total) return;
    const int d = (D > 0) ? D : m.d;
    const int nch = m.C / d;
    int rr = (int)(gi / nch);
    int j = (int)(gi - (int64_t)rr * nch);
    int r = r0 + rr;
    const uint32_t K = 1u << m.bits;
    uint32_t tag = cbl_read_tag(m.tags + (int64_t)r * m.W, m.W, j, m.bits);
    if (m.row_book) tag += (uint32_t)m.row_book[r] * K;
    const __half* cw = (const __half*)m.table + (int64_t)tag * d;
    const __half* cw2 = nullptr;
    if (m.books == 2) cw2 = (const __half*)m.table2 + (int64_t)cbl_read_tag(m.tags2 + (int64_t)r * m.W, m.W, j, m.bits) * d;
    const float rs = __half2float(((const __half*)m.row_scale)[r]);
    const int32_t* perm = (m.M > 1) ? m.perms + (int64_t)m.row_mask[r] * m.C : nullptr;
    OutT* orow = out + (int64_t)rr * ld;
    if (VEC && D == 8) {
        // M == 1, 8 values per chunk: one 16-byte table read, contiguous aligned stores
        uint4 q = __ldg((const uint4*)cw);
        const __half2* h = (const __half2*)&q;
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
        if (cw2) {
            uint4 q2 = __ldg((const uint4*)cw2);
            const __half2* h2 = (const __half2*)&q2;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __half22float2(h2[i]);
                v[2 * i] = __fadd_rn(v[2 * i], f.x);
                v[2 * i + 1] = __fadd_rn(v[2 * i + 1], f.y);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(v[i], rs);
        OutT* o = orow + j * 8;
        if (sizeof(OutT) == 4) {
            float4* o4 = (float4*)o;
            o4[0] = make_float4(v[0], v[1], v[2], v[3]);
            o4[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
            union { uint4 u; OutT t[8]; } pk;
#pragma unroll
            for (int i = 0; i < 8; i++) pk.t[i] = cbl_cvt_out<OutT>(v[i]);
            *(uint4*)o = pk.u;
        }
    } else {
        for (int i = 0; i < d; i++) {
            float u = __half2float(cw[i]);
            if (cw2) u = __fadd_rn(u, __half2float(cw2[i]));
            u = __fmul_rn(u, rs);
            int c = j * d + i;
            if (perm) c = perm[c];
            orow[c] = cbl_cvt_out<OutT>(u);
        }
    }
}

// The benchmark format (d = 8, 12-bit tags, one table per book, one column order) and at least a few hundred rows: the
// book(s) live in shared memory, a warp walks a row 256 chunks at a time (tags straight from the row's bit stream, one
// 16-byte codeword read per chunk, one 16- or 32-byte store), same arithmetic as k_dequant.  HBM-write bound.
constexpr int DQ_THREADS = 512;
template <typename OutT, int BOOKS>
__global__ void __launch_bounds__(DQ_THREADS, 2) k_dequant_book(cbl_packed m, OutT* __restrict__ out, int64_t ld, int r0, int r1) {
    extern __shared__ __align__(16) unsigned char dq_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    {
        uint4* dst = (uint4*)dq_smem;
        const uint4* t0 = (const uint4*)m.table;
        for (int i = tid; i < 4096; i += DQ_THREADS) dst[i] = __ldg(t0 + i);
        if (BOOKS == 2) {
            const uint4* t1 = (const uint4*)m.table2;
            for (int i = tid; i < 4096; i += DQ_THREADS) dst[4096 + i] = __ldg(t1 + i);
        }
    }
    __syncthreads();
    const uint32_t sb = cbl_smem_u32(dq_smem);
    const int nch = m.C >> 3;
    constexpr int NB = (sizeof(OutT) == 2 && BOOKS == 1) ? 8 : 4;   // chunks per lane in flight
    auto tag_of = [&](const int32_t* rw, int j) {
        const uint32_t bit = 12u * (uint32_t)j, w = bit >> 5, sh = bit & 31u;
        const uint32_t lo = (uint32_t)__ldg(rw + w);
        const uint32_t hi = (sh > 20u && (int)(w + 1) < m.W) ? (uint32_t)__ldg(rw + w + 1) : 0u;
        return (__funnelshift_r(lo, hi, sh) & 0xFFFu) << 4;
    };
    for (int r = r0 + blockIdx.x * (DQ_THREADS / 32) + warp; r < r1; r += gridDim.x * (DQ_THREADS / 32)) {
        const int32_t* rw = m.tags + (int64_t)r * m.W;
        const int32_t* rw2 = BOOKS == 2 ? m.tags2 + (int64_t)r * m.W : nullptr;
        const float rs = __half2float(((const __half*)m.row_scale)[r]);
        OutT* orow = out + (int64_t)(r - r0) * ld;
        for (int j0 = 0; j0 < nch; j0 += 32 * NB) {
            uint4 cw[NB], cw2[BOOKS == 2 ? NB : 1];
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const int j = j0 + 32 * i + lane;
                cw[i] = make_uint4(0, 0, 0, 0);
                if (j < nch) {
                    cw[i] = cbl_lds128(sb + tag_of(rw, j));
                    if (BOOKS == 2) cw2[i] = cbl_lds128(sb + 65536u + tag_of(rw2, j));
                }
            }
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const int j = j0 + 32 * i + lane;
                if (j >= nch) continue;
                const __half2* h = (const __half2*)&cw[i];
                float v[8];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(h[e]);
                    v[2 * e] = f.x;
                    v[2 * e + 1] = f.y;
                }
                if (BOOKS == 2) {
                    const __half2* h2 = (const __half2*)&cw2[i];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(h2[e]);
                        v[2 * e] = __fadd_rn(v[2 * e], f.x);
                        v[2 * e + 1] = __fadd_rn(v[2 * e + 1], f.y);
                    }
                }
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], rs);
                OutT* o = orow + j * 8;
                if (sizeof(OutT) == 4) {
                    float4* o4 = (float4*)o;
                    o4[0] = make_float4(v[0], v[1], v[2], v[3]);
                    o4[1] = make_float4(v[4], v[5], v[6], v[7]);
                } else {
                    uint4 pk;                                      // two values per conversion instruction
                    uint32_t* pw = (uint32_t*)&pk;
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if (std::is_same<OutT, __half>::value) {
                            const __half2 h2 = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                            pw[e] = *(const uint32_t*)&h2;
                        } else {
                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                            pw[e] = *(const uint32_t*)&b2;
                        }
                    }
                    *(uint4*)o = pk;
                }
            }
        }
    }
}

template <typename OutT, int BOOKS>
static int launch_dequant_book(const cbl_packed* m, void* out, int64_t ld, int r0, int r1, cudaStream_t st) {
    const size_t smem = (size_t)BOOKS * 65536;
    static bool attr_set[64] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        CBL_CUDA(cudaFuncSetAttribute(k_dequant_book<OutT, BOOKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    int grid = cbl_sm_count() * (BOOKS == 1 ? 2 : 1);
    const int need = cbl_ceil_div(r1 - r0, DQ_THREADS / 32);
    if (grid > need) grid = need;
    k_dequant_book<OutT, BOOKS><<<grid, DQ_THREADS, smem, st>>>(*m, (OutT*)out, ld, r0, r1);
    return cbl_check_launch();
}

template <typename OutT>
static int launch_dequant(const cbl_packed* m, void* out, int64_t ld, int r0, int r1, cudaStream_t st) {
    int64_t n = (int64_t)(r1 - r0) * (m->C / m->d);
    if (n == 0) return CBL_OK;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return CBL_EUNSUPPORTED;
    bool vec = m->M == 1 && m->d == 8 && (ld % 8 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)m->table % 16 == 0) &&
               (m->books == 1 || (uintptr_t)m->table2 % 16 == 0);
    // enough rows to pay for staging the book(s) in every block: the shared-memory kernel
#ifdef CBL_DEQUANT_GENERIC
    const bool generic = true;                                 // build option: always the generic kernel (comparisons)
#else
    const bool generic = false;
#endif
    if (!generic && vec && m->bits == 12 && m->G == 1 && !m->row_book && (int64_t)(r1 - r0) * m->C >= (1 << 22)) {
        if (m->books == 1) return launch_dequant_book<OutT, 1>(m, out, ld, r0, r1, st);
        return launch_dequant_book<OutT, 2>(m, out, ld, r0, r1, st);
    }
    if (vec) k_dequant<OutT, 8, true><<<(unsigned)blocks, 256, 0, st>>>(*m, (OutT*)out, ld, r0, n);
    else k_dequant<OutT, 0, false><<<(unsigned)blocks, 256, 0, st>>>(*m, (OutT*)out, ld, r0, n);
    return cbl_check_launch();
}

extern "C" int cbl_dequant(const cbl_packed* m, void* out, int dtype, int64_t ld, int32_t r0, int32_t r1, cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (r0 < 0 || r1 < r0 || r1 > m->R || ld < m->C) return CBL_EINVAL;
    if (r0 == r1) return CBL_OK;
    if (!out) return CBL_EINVAL;
    cudaStream_t st = (cudaStream_t)s;
    switch (dtype) {
        case CBL_F32: return launch_dequant<float>(m, out, ld, r0, r1, st);
        case CBL_F16: return launch_dequant<__half>(m, out, ld, r0, r1, st);
        case CBL_BF16: return launch_dequant<__nv_bfloat16>(m, out, ld, r0, r1, st);
        default: return CBL_EINVAL;
    }
}

// ------------------------------------------------------------------------------------ tags
__global__ void __launch_bounds__(256) k_unpack(cbl_packed m, const int32_t* __restrict__ words, int32_t* __restrict__ out, int64_t n) {
    int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= n) return;
    int nch = m.C / m.d;
    int r = (int)(gi / nch), j = (int)(gi - (int64_t)r * nch);
    out[gi] = (int32_t)cbl_read_tag(words + (int64_t)r * m.W, m.W, j, m.bits);
}

extern "C" int cbl_unpack_tags(const cbl_packed* m, int plane, int32_t* out, cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (!out || plane < 0 || plane >= m->books) return CBL_EINVAL;
    int64_t n = (int64_t)m->R * (m->C / m->d);
    if (n == 0) return CBL_OK;
    k_unpack<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)s>>>(*m, plane ? m->tags2 : m->tags, out, n);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ t16 layout
//
// Lane (g = lane >> 2, t = lane & 3) of the warp that owns a 16-row tile multiplies rows g and
// g + 8; in step s of a super-step it takes chunk column (ss*16 + s)*4 + t.  Its 32 tags of one
// super-step (i = 2*s + h, h = 0: row g, h = 1: row g + 8) form a 384-bit little-endian stream
// stored as three uint4 at [book][tile][ss][q][lane].
static int t16_nsuper(int C) { return cbl_ceil_div(C / 8, 64); }

extern "C" size_t cbl_t16_bytes(int32_t ntile, int32_t C, int32_t books) {
    if (ntile < 0 || C <= 0 || books < 1) return 0;
    return (size_t)books * ntile * t16_nsuper(C) * 3 * 32 * 16;
}

__global__ void __launch_bounds__(128) k_repack_t16(cbl_packed m, const int32_t* __restrict__ tile_rows, int ntile, int nsuper,
                                                    uint4* __restrict__ out, int64_t nthreads) {
    int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= nthreads) return;
    int lane = (int)(gi & 31);
    int64_t rest = gi >> 5;
    int ss = (int)(rest % nsuper);
    rest /= nsuper;
    int tile = (int)(rest % ntile);
    int book = (int)(rest / ntile);
    int g = lane >> 2, t = lane & 3;
    const int nch = m.C / 8;
    const int32_t* words = book ? m.tags2 : m.tags;
    int rows[2] = {tile_rows[tile * 16 + g], tile_rows[tile * 16 + g + 8]};
    uint32_t w[13];
#pragma unroll
    for (int i = 0; i < 13; i++) w[i] = 0;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        int sidx = i >> 1, h = i & 1;
        int chunk = (ss * 16 + sidx) * 4 + t;
        uint32_t tag = 0;
        if (rows[h] >= 0 && chunk < nch) tag = cbl_read_tag(words + (int64_t)rows[h] * m.W, m.W, chunk, 12);
        int bit = 12 * i;
        w[bit >> 5] |= tag << (bit & 31);
        if ((bit & 31) > 20) w[(bit >> 5) + 1] |= tag >> (32 - (bit & 31));
    }
    uint4* o = out + (((int64_t)book * ntile + tile) * nsuper + ss) * 96 + lane;
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[32] = make_uint4(w[4], w[5], w[6], w[7]);
    o[64] = make_uint4(w[8], w[9], w[10], w[11]);
}

extern "C" int cbl_repack_t16(const cbl_packed* m, const int32_t* tile_rows, int32_t ntile, void* out, cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (m->d != 8 || m->bits != 12 || m->G != 1) return CBL_EUNSUPPORTED;
    if (!tile_rows || !out || ntile < 0 || ((uintptr_t)out % 16)) return CBL_EINVAL;
    int nsuper = t16_nsuper(m->C);
    int64_t n = (int64_t)m->books * ntile * nsuper * 32;
    if (n == 0) return CBL_OK;
    k_repack_t16<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)s>>>(*m, tile_rows, ntile, nsuper, (uint4*)out, n);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ x16 layout
//
// Column range kr = chunks 16 kr .. 16 kr + 15, row block rb = rows 64 rb .. 64 rb + 63.  Lane (g, t) of a warp owns,
// for each of the block's 8 row tiles rt, the 4 chunks 16 kr + 4 j + t (j = 0..3) of row 64 rb + 8 rt + g: 32 tags,
// tag index 4 rt + j, packed as a 384-bit little-endian stream = three uint4 at [book][kr][rb][3][32 lanes].
extern "C" size_t cbl_x16_bytes(int32_t R, int32_t C, int32_t books) {
    if (R < 0 || C <= 0 || books < 1) return 0;
    return (size_t)books * cbl_ceil_div(C / 8, 16) * cbl_ceil_div(R, 64) * 96 * 16;
}

__global__ void __launch_bounds__(128) k_repack_x16(cbl_packed m, int nkr, int nrb, uint4* __restrict__ out, int64_t nthreads) {
    int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= nthreads) return;
    const int lane = (int)(gi & 31);
    int64_t rest = gi >> 5;
    const int rb = (int)(rest % nrb);
    rest /= nrb;
    const int kr = (int)(rest % nkr);
    const int book = (int)(rest / nkr);
    const int g = lane >> 2, t = lane & 3;
    const int nch = m.C / 8;
    const int32_t* words = book ? m.tags2 : m.tags;
    uint32_t w[13];
#pragma unroll
    for (int i = 0; i < 13; i++) w[i] = 0;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const int rt = i >> 2, j = i & 3;
        const int row = rb * 64 + rt * 8 + g, chunk = kr * 16 + 4 * j + t;
        uint32_t tag = 0;
        if (row < m.R && chunk < nch) tag = cbl_read_tag(words + (int64_t)row * m.W, m.W, chunk, 12);
        const int bit = 12 * i;
        w[bit >> 5] |= tag << (bit & 31);
        if ((bit & 31) > 20) w[(bit >> 5) + 1] |= tag >> (32 - (bit & 31));
    }
    uint4* o = out + (((int64_t)book * nkr + kr) * nrb + rb) * 96 + lane;
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[32] = make_uint4(w[4], w[5], w[6], w[7]);
    o[64] = make_uint4(w[8], w[9], w[10], w[11]);
}

extern "C" int cbl_repack_x16(const cbl_packed* m, void* out, cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (m->d != 8 || m->bits != 12 || m->G != 1 || m->M != 1) return CBL_EUNSUPPORTED;
    if (!out || ((uintptr_t)out % 16)) return CBL_EINVAL;
    const int nkr = cbl_ceil_div(m->C / 8, 16), nrb = cbl_ceil_div(m->R, 64);
    const int64_t n = (int64_t)m->books * nkr * nrb * 32;
    if (n == 0) return CBL_OK;
    k_repack_x16<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)s>>>(*m, nkr, nrb, (uint4*)out, n);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ l8 layout
//
// Tile v covers chunk columns 8*(v % ntile1) .. +7 of book v / ntile1.  Row r's 8 tags of the tile
// form a 96-bit little-endian stream; word k of that stream is stored at [v][k][r], so that four
// consecutive rows' k-th words are one aligned 128-bit load.
extern "C" size_t cbl_l8_bytes(int32_t R, int32_t C, int32_t books) {
    if (R < 0 || C <= 0 || books < 1) return 0;
    size_t Rpad = ((size_t)R + 3) / 4 * 4;
    return (size_t)books * cbl_ceil_div(C / 8, 8) * 3 * Rpad * 4;
}

__global__ void __launch_bounds__(256) k_repack_l8(cbl_packed m, int ntile1, int Rpad, uint32_t* __restrict__ out, int64_t nthreads) {
    int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= nthreads) return;
    int r = (int)(gi % Rpad);
    int v = (int)(gi / Rpad);
    int book = v / ntile1, tile = v % ntile1;
    const int nch = m.C / 8;
    const int32_t* words = book ? m.tags2 : m.tags;
    uint32_t w[4] = {0, 0, 0, 0};
    if (r < m.R) {
#pragma unroll
        for (int c = 0; c < 8; c++) {
            int chunk = tile * 8 + c;
            uint32_t tag = chunk < nch ? cbl_read_tag(words + (int64_t)r * m.W, m.W, chunk, 12) : 0u;
            int bit = 12 * c;
            w[bit >> 5] |= tag << (bit & 31);
            if ((bit & 31) > 20) w[(bit >> 5) + 1] |= tag >> (32 - (bit & 31));
        }
    }
    uint32_t* o = out + (int64_t)v * 3 * Rpad + r;
    o[0] = w[0];
    o[Rpad] = w[1];
    o[2 * (int64_t)Rpad] = w[2];
}

extern "C" int cbl_repack_l8(const cbl_packed* m, void* out, cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (m->d != 8 || m->bits != 12 || m->G != 1 || m->M != 1) return CBL_EUNSUPPORTED;
    if (!out || ((uintptr_t)out % 16)) return CBL_EINVAL;
    int ntile1 = cbl_ceil_div(m->C / 8, 8);
    int Rpad = (m->R + 3) / 4 * 4;
    int64_t n = (int64_t)m->books * ntile1 * Rpad;
    if (n == 0) return CBL_OK;
    k_repack_l8<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)s>>>(*m, ntile1, Rpad, (uint32_t*)out, n);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ product for every format the file layout can hold
//
// y[t, r] = round(row_scale[r] * sum_j <table[row_book[r] * K + tag(r, j)] (+ table2[tag2(r, j)]), x[t, perms[row_mask[r]][j d .. j d + d)]>)
// for any chunk length d <= 16, tag width <= 16 bits, several books per matrix (row_book) and several column orders:
// the formats the reference's generic kernel executes and the table-lookup / tensor-core kernels here do not.  A
// warp per row: its lanes take every 32nd chunk, read the codeword from the L1/L2-resident table and the chunk's
// activations through the row's column order, and accumulate up to GEN_TOK tokens in fp32; shuffles add the lanes.
// Not a bandwidth kernel: correctness for the formats outside the benchmark's.
constexpr int GEN_TOK = 4;
__global__ void __launch_bounds__(256) k_gemv_generic(cbl_packed m, const void* __restrict__ x, int xdtype, int ntok, int64_t ldx,
                                                      void* __restrict__ y, int ydtype, int64_t ldy) {
    const int lane = threadIdx.x & 31, r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= m.R) return;
    const int d = m.d, nch = m.C / d;
    const uint32_t K = 1u << m.bits, boff = m.row_book ? (uint32_t)m.row_book[r] * K : 0u;
    const int32_t* rw = m.tags + (int64_t)r * m.W;
    const int32_t* rw2 = m.books == 2 ? m.tags2 + (int64_t)r * m.W : nullptr;
    const int32_t* perm = m.M > 1 ? m.perms + (int64_t)m.row_mask[r] * m.C : nullptr;
    const float rs = __half2float(((const __half*)m.row_scale)[r]);
    for (int t0 = 0; t0 < ntok; t0 += GEN_TOK) {
        float acc[GEN_TOK];
#pragma unroll
        for (int t = 0; t < GEN_TOK; t++) acc[t] = 0.f;
        for (int j = lane; j < nch; j += 32) {
            const __half* cw = (const __half*)m.table + (int64_t)(boff + cbl_read_tag(rw, m.W, j, m.bits)) * d;
            const __half* cw2 = rw2 ? (const __half*)m.table2 + (int64_t)cbl_read_tag(rw2, m.W, j, m.bits) * d : nullptr;
            for (int i = 0; i < d; i++) {
                float w = __half2float(cw[i]);
                if (cw2) w = __fadd_rn(w, __half2float(cw2[i]));          // the decode's order: the two codewords are added first
                const int c = perm ? perm[j * d + i] : j * d + i;
#pragma unroll
                for (int t = 0; t < GEN_TOK; t++)
                    if (t0 + t < ntok) acc[t] = fmaf(w, cbl_load_in(x, xdtype, (int64_t)(t0 + t) * ldx + c), acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < GEN_TOK; t++) {
            float v = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && t0 + t < ntok) cbl_store_out(y, ydtype, (int64_t)(t0 + t) * ldy + r, v * rs);
        }
    }
}

extern "C" int cbl_gemv_generic(const cbl_packed* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                                cbl_stream s) {
    int rc = check_packed(m);
    if (rc) return rc;
    if (!x || !y || ntok < 0 || ldy < m->R) return CBL_EINVAL;
    if (xdtype != CBL_F32 && xdtype != CBL_F16 && xdtype != CBL_BF16) return CBL_EINVAL;
    if (ydtype != CBL_F32 && ydtype != CBL_F16 && ydtype != CBL_BF16) return CBL_EINVAL;
    if (m->R == 0 || ntok == 0) return CBL_OK;
    k_gemv_generic<<<cbl_ceil_div(m->R, 8), 256, 0, (cudaStream_t)s>>>(*m, x, xdtype, ntok, ldx, y, ydtype, ldy);
    return cbl_check_launch();
}
