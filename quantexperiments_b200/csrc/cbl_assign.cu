// Encoder side of the format: nearest codeword of every 8-wide chunk (the "snap" that produces the tags) and the
// little-endian bit packing of the tags.
//
// k_assign     each thread keeps CH chunks in registers and scans the whole book from shared memory (fp32, read as
//              warp-wide broadcasts): 8 fp32 FMAs per (chunk, codeword) starting from |c|^2, i.e. c_sq - 2 x.c in fp32
//              exactly as the reference states it.  The minimum is tracked per group of eight codewords (one min per
//              codeword and one compare per group instead of a compare and two selects per codeword); the winning
//              group is evaluated once more at the end to name the first codeword that reaches the minimum.
//              Bound by the fp32 FMA rate, not by memory: 65 kflop per 44 bytes of traffic.
// k_pack_tags  one thread per 32-bit word of the stream.
#include "cbl_common.cuh"
#include <cmath>

constexpr int AS_THREADS = 256, AS_GROUP = 8;

// Three-input minimum (one instruction on sm_100).
__device__ __forceinline__ float as_min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

template <int CH, bool WT>
__global__ void __launch_bounds__(AS_THREADS, 1)
k_assign(const float* __restrict__ x, const float* __restrict__ wt, int64_t n, const void* __restrict__ book, int bdtype, int K, int Kpad,
         int64_t* __restrict__ idx, float* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char as_smem[];
    float4* s_book = (float4*)as_smem;                       // [Kpad][2]
    float* s_init = (float*)(as_smem + (size_t)Kpad * 32);   // |c|^2 (0 when weighted); +inf for the padding
    const int tid = threadIdx.x;
    for (int k = tid; k < Kpad; k += AS_THREADS) {
        float c[8], sq = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            c[i] = k < K ? cbl_load_in(book, bdtype, (int64_t)k * 8 + i) : 0.f;
            sq += c[i] * c[i];
        }
        s_book[2 * k] = make_float4(c[0], c[1], c[2], c[3]);
        s_book[2 * k + 1] = make_float4(c[4], c[5], c[6], c[7]);
        s_init[k] = k < K ? (WT ? 0.f : sq) : INFINITY;
    }
    __syncthreads();
    const int64_t per_block = (int64_t)AS_THREADS * CH;
    for (int64_t base = (int64_t)blockIdx.x * per_block; base < n; base += (int64_t)gridDim.x * per_block) {
        float a[CH][8], w[WT ? CH : 1][8], xx[CH], best[CH];
        int bg[CH];
#pragma unroll
        for (int j = 0; j < CH; j++) {
            const int64_t ci = base + (int64_t)j * AS_THREADS + tid;
            float4 lo = make_float4(0, 0, 0, 0), hi = lo, wl = lo, wh = lo;
            if (ci < n) {
                lo = __ldg((const float4*)x + 2 * ci);
                hi = __ldg((const float4*)x + 2 * ci + 1);
                if (WT) { wl = __ldg((const float4*)wt + 2 * ci); wh = __ldg((const float4*)wt + 2 * ci + 1); }
            }
            const float xv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const float wv[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (WT) {
                    w[j][i] = wv[i];
                    a[j][i] = (-2.0f * wv[i]) * xv[i];
                    s += (wv[i] * xv[i]) * xv[i];
                } else {
                    a[j][i] = -2.0f * xv[i];
                    s += xv[i] * xv[i];
                }
            }
            xx[j] = s;
            best[j] = INFINITY;
            bg[j] = 0;
        }
        auto dist = [&](int j, const float4& c0, const float4& c1, float init) -> float {
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            float d = init;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (WT) d = fmaf(c[i], fmaf(w[j][i], c[i], a[j][i]), d);
                else d = fmaf(a[j][i], c[i], d);
            }
            return d;
        };
        for (int k0 = 0; k0 < Kpad; k0 += AS_GROUP) {
            float gm[CH];
#pragma unroll
            for (int j = 0; j < CH; j++) gm[j] = INFINITY;
#pragma unroll
            for (int q = 0; q < AS_GROUP; q += 2) {
                const float4 c0 = s_book[2 * (k0 + q)], c1 = s_book[2 * (k0 + q) + 1];
                const float4 e0 = s_book[2 * (k0 + q) + 2], e1 = s_book[2 * (k0 + q) + 3];
                const float2 init = *(const float2*)(s_init + k0 + q);
#pragma unroll
                for (int j = 0; j < CH; j++) gm[j] = as_min3(gm[j], dist(j, c0, c1, init.x), dist(j, e0, e1, init.y));
            }
#pragma unroll
            for (int j = 0; j < CH; j++)
                if (gm[j] < best[j]) { best[j] = gm[j]; bg[j] = k0; }
        }
#pragma unroll
        for (int j = 0; j < CH; j++) {
            const int64_t ci = base + (int64_t)j * AS_THREADS + tid;
            if (ci >= n) continue;
            int bi = bg[j];
            float bd = INFINITY;
#pragma unroll
            for (int q = 0; q < AS_GROUP; q++) {
                const int k = bg[j] + q;
                const float dq = dist(j, s_book[2 * k], s_book[2 * k + 1], s_init[k]);
                if (dq < bd) { bd = dq; bi = k; }
            }
            idx[ci] = bi < K ? bi : 0;
            err[ci] = fmaxf(bd + xx[j], 0.f);
        }
    }
}

extern "C" int cbl_assign_max_codewords() { return 4096; }

extern "C" int cbl_assign(const float* x, const float* wt, int64_t n, int32_t d, const void* book, int bdtype, int32_t K, int64_t* idx,
                          float* err, cbl_stream s) {
    if (!book || n < 0 || K < 1 || (n > 0 && (!x || !idx || !err))) return CBL_EINVAL;
    if (bdtype != CBL_F16 && bdtype != CBL_BF16 && bdtype != CBL_F32) return CBL_EINVAL;
    if (d != 8 || K > 4096) return CBL_EUNSUPPORTED;
    if (((uintptr_t)x % 16) || (wt && ((uintptr_t)wt % 16))) return CBL_EINVAL;
    if (n == 0) return CBL_OK;
    const int Kpad = (K + AS_GROUP - 1) / AS_GROUP * AS_GROUP;
    const size_t smem = (size_t)Kpad * 36;
    static bool attr_set[64][2] = {};
    int dev = 0;
    CBL_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev][wt ? 1 : 0]) {
        if (wt) CBL_CUDA(cudaFuncSetAttribute(k_assign<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4096 * 36));
        else CBL_CUDA(cudaFuncSetAttribute(k_assign<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4096 * 36));
        attr_set[dev][wt ? 1 : 0] = true;
    }
    const int ch = wt ? 4 : 8;
    int64_t blocks = (n + (int64_t)AS_THREADS * ch - 1) / ((int64_t)AS_THREADS * ch);
    const int sms = cbl_sm_count();
    // whole waves: every block scans the same number of chunk batches (the last may be short)
    if (blocks > sms) blocks = sms;
    if (wt) k_assign<4, true><<<(unsigned)blocks, AS_THREADS, smem, (cudaStream_t)s>>>(x, wt, n, book, bdtype, K, Kpad, idx, err);
    else k_assign<8, false><<<(unsigned)blocks, AS_THREADS, smem, (cudaStream_t)s>>>(x, wt, n, book, bdtype, K, Kpad, idx, err);
    return cbl_check_launch();
}

// ------------------------------------------------------------------------------------ bit packing
__global__ void __launch_bounds__(256) k_pack_tags(const int64_t* __restrict__ vals, int64_t R, int n, int bits, int W, int32_t* __restrict__ words) {
    const int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= R * W) return;
    const int64_t r = gi / W;
    const int wi = (int)(gi % W);
    const int64_t b0 = (int64_t)wi * 32;
    const unsigned long long mask = (1ull << bits) - 1ull;
    unsigned int out = 0;
    for (int t = (int)(b0 / bits); t < n && (int64_t)t * bits < b0 + 32; t++) {
        const unsigned long long v = (unsigned long long)vals[r * n + t] & mask;
        const int64_t sh = (int64_t)t * bits - b0;          // position of the tag's bit 0 relative to the word
        out |= sh >= 0 ? (unsigned int)(v << sh) : (unsigned int)(v >> (-sh));
    }
    words[gi] = (int32_t)out;
}

extern "C" int cbl_pack_tags(const int64_t* vals, int64_t R, int32_t n, int32_t bits, int32_t* words, cbl_stream s) {
    if (!vals || !words || R < 0 || n < 1 || bits < 1 || bits > 16) return CBL_EINVAL;
    const int W = (int)(((int64_t)n * bits + 31) / 32);
    const int64_t total = R * W;
    if (total == 0) return CBL_OK;
    k_pack_tags<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)s>>>(vals, R, n, bits, W, words);
    return cbl_check_launch();
}
