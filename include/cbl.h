/*
 * cbl.h - C ABI of libcbl: the codebook-linear hot path on B200 (sm_100a).
 *
 * The library executes one storage format: an [R, C] weight matrix cut into chunks of d values
 * along the input dimension, every chunk replaced by a log2(K)-bit tag into a table of fp16
 * codewords, an fp16 scale per row, optionally a second summed table ("additive" books) and
 * per-row seeded column orders.  The format is the one defined by the reference project
 * angryslavemerchant/QuantExperiments in shapequant/packed.py:1-27.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless a comment says otherwise; plain C types only;
 *   - every function returns an int status: CBL_OK or a negative cbl_status; nothing throws,
 *     traps or aborts, and nothing allocates or frees device memory: the caller owns all
 *     buffers and passes work space explicitly (sizes come from the *_bytes() queries);
 *   - work is enqueued on the CUDA stream given (a cudaStream_t cast to cbl_stream); functions
 *     return after the launch, they do not synchronise;
 *   - a reference citation "replaces file:line" names the reference function whose role the
 *     entry point takes (paths are inside the reference repository).
 */
#ifndef CBL_H
#define CBL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* cbl_stream;

typedef enum cbl_status {
    CBL_OK = 0,
    CBL_EINVAL = -1,        /* bad argument (null pointer, negative size, misaligned buffer) */
    CBL_EUNSUPPORTED = -2,  /* a shape or format variant this kernel does not execute */
    CBL_ECUDA = -3,         /* a CUDA runtime call failed; cbl_last_cuda_error() has the code */
    CBL_ETIMEOUT = -4       /* a bounded device-side wait expired (reported by status words) */
} cbl_status;

typedef enum cbl_dtype { CBL_F32 = 0, CBL_F16 = 1, CBL_BF16 = 2 } cbl_dtype;

/* Library version (major*10000 + minor*100 + patch) and the SM architecture it was built for. */
int cbl_version(void);
int cbl_built_for_sm(void);
const char* cbl_status_string(int status);
int cbl_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * The file layout (device copy of the tensors of one matrix, shapequant/packed.py:8-16):
 *   tags      int32 [R, W]    little-endian bit stream of `bits`-bit tags per row, W words
 *   table     fp16  [G*K, d]  codewords
 *   row_scale fp16  [R]
 *   row_book  uint8 [R]       codebook of each row, or NULL when G == 1
 *   row_mask  uint8 [R]       column order of each row, or NULL when M == 1
 *   perms     int32 [M, C]    the column orders (regenerated from the seed on the host), or NULL
 * books == 2 adds a second tag plane and table whose codewords are summed with the first
 * (tests/test_proto_runs.py:135-144 of the reference); G must be 1 in that case.
 * ------------------------------------------------------------------------------------------ */
typedef struct cbl_packed {
    int32_t R, C, d, bits, G, M, books, W;
    const int32_t* tags;
    const int32_t* tags2;
    const void* table;
    const void* table2;
    const void* row_scale;
    const uint8_t* row_book;
    const uint8_t* row_mask;
    const int32_t* perms;
} cbl_packed;

/* Dense decode of rows [r0, r1) into out[(r - r0) * ld + c], c in the original column order:
 *   u = fp32(table[row_book[r]*K + tag]) (+ fp32(table2[tag2]))   rounded to fp32
 *   w[r, perms[row_mask[r]][j*d + i]] = round_to(dtype, u * fp32(row_scale[r]))
 * Bit-exact with the reference decode for f32 and one round-to-nearest of it for f16 / bf16.
 * Any d in 1..16, bits in 1..16.
 * replaces shapequant/packed.py:259-270 (decode_tensors), shapequant/codebook.py:277-289 (decode),
 *          shapequant/kernels/cuda_dequant.py:79-103 (dequant, incl. its rows=(r0, r1) range),
 *          shapequant/kernels/batched_runs.py:935-961 (dequant_tile, fp16 / bf16 output). */
int cbl_dequant(const cbl_packed* m, void* out, int dtype, int64_t ld, int32_t r0, int32_t r1, cbl_stream s);

/* Product for EVERY format the file layout can hold (any d <= 16, tags of up to 16 bits, several books per matrix
 * through row_book, one or two summed books, several column orders), the formats outside the benchmark's d = 8 /
 * 12-bit / one-book-per-matrix that the table-lookup and tensor-core kernels execute:
 *   y[t * ldy + r] = round(row_scale[r] * sum_c W[r, c] * x[t * ldx + c]),  W = the decode above without the row scale
 * fp32 accumulate; x f32 / f16 / bf16 (a column shard with column orders may index beyond C: ldx covers the vector),
 * y f32 / f16 / bf16.  A correctness path (a warp per row, codewords from the cache-resident table), not a bandwidth
 * kernel.
 * replaces shapequant/kernels/gemv.py:28-64 (_gemv_kernel: any d, book_off, row_mask / perms) for those formats. */
int cbl_gemv_generic(const cbl_packed* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                     cbl_stream s);

/* Encoder side ("snap"): index of the nearest codeword of every chunk and its squared error,
 *   idx[i] = argmin_k (|c_k|^2 - 2 x_i . c_k)   (first k on ties),   err[i] = max(min + |x_i|^2, 0),
 * all in fp32 (8 FMAs per codeword from |c_k|^2, no reduced-precision contraction).  wt (optional, same shape as x):
 * per-element weights, argmin_k sum_j wt_j (x_j - c_kj)^2 and err = that minimum.
 * x, wt fp32 [n, d]; book f16 / bf16 / f32 [K, d]; d = 8, K <= cbl_assign_max_codewords().
 * replaces shapequant/codebook.py:40-71 (_assign_batch, assign). */
int cbl_assign_max_codewords(void);
int cbl_assign(const float* x, const float* wt, int64_t n, int32_t d, const void* book, int bdtype, int32_t K, int64_t* idx, float* err,
               cbl_stream s);

/* [R, n] tags (low `bits` bits of each int64) -> [R, ceil(n * bits / 32)] int32, a little-endian bit stream per row.
 * replaces shapequant/packed.py:60-77 (pack_bits). */
int cbl_pack_tags(const int64_t* vals, int64_t R, int32_t n, int32_t bits, int32_t* words, cbl_stream s);

/* Unpacked tags of plane `plane` (0 or 1) as int32 [R, C/d].
 * replaces shapequant/packed.py:80-90 (unpack_bits) / :246-248 (PackedFile.local_tags). */
int cbl_unpack_tags(const cbl_packed* m, int plane, int32_t* out, cbl_stream s);

/* ------------------------------------------------------------------------------------------
 * Row-tile layout ("t16") for the small-batch product: rows are grouped by column order into
 * tiles of 16 (tile_rows[tile*16 + i] = source row or -1), tags re-ordered so that every lane of
 * a warp reads its own tags with 128-bit loads.  d = 8, bits = 12, G = 1 only.
 * replaces shapequant/kernels/batched_runs.py:643-677 (tile_words) and
 *          shapequant/kernels/proto_runs.py:322-336, 380-388 (pack_lane_major, make_tiles).
 * ------------------------------------------------------------------------------------------ */
typedef struct cbl_t16 {
    int32_t R, C, books, M, ntile, nsuper;
    const void* words;         /* uint4 [books][ntile][nsuper][3][32] */
    const int32_t* tile_rows;  /* [ntile * 16], -1 = padding row */
    const int32_t* tile_mask;  /* [ntile] column order of the tile, NULL when M == 1 */
    const void* table;         /* fp16 [4096, 8] */
    const void* table2;        /* fp16 [4096, 8] when books == 2 */
    const void* row_scale;     /* fp16 [R], indexed by source row */
} cbl_t16;

size_t cbl_t16_bytes(int32_t ntile, int32_t C, int32_t books);
int cbl_repack_t16(const cbl_packed* m, const int32_t* tile_rows, int32_t ntile, void* out, cbl_stream s);

/* Activations for cbl_gemv_t16: x [B, C] (row stride ldx, f16 or bf16) -> xp fp16
 * [M][Bpad][Cpad] with xp[m][b][c] = x[b][perms[m][c]], zero padded (Bpad = B rounded up to 8,
 * Cpad = C rounded up to 512).
 * replaces shapequant/kernels/proto_runs.py:500-502 (prep_x). */
size_t cbl_prep_x_bytes(int32_t B, int32_t C, int32_t M);
int cbl_prep_x(const void* x, int xdtype, int32_t B, int32_t C, int64_t ldx, const int32_t* perms, int32_t M,
               void* xp, cbl_stream s);

/* y[b*ldy + r] = round_to(ydtype, row_scale[r] * sum_c W[r, c] * x[b, c]) for b < B <= 64,
 * tensor-core (mma.sync) product with fp32 accumulation straight from the packed tags.
 * replaces shapequant/kernels/batched_runs.py:745-771 (RunsBatch.run) and, for B = 1 with column
 *          orders or two books, shapequant/kernels/proto_runs.py:412-473, 505-571 (gemv_additive, gemv). */
int cbl_gemv_t16(const cbl_t16* m, const void* xp, int32_t B, void* y, int ydtype, int64_t ldy, cbl_stream s);

/* ------------------------------------------------------------------------------------------
 * Column-tile layout ("l8"): a tile = 8 chunk columns (64 weight columns); the 8 tags of a row and tile
 * form a 96-bit stream, word k of it stored at [tile][k][row position] (books = 2: a second run of tiles).
 * Two variants share the struct:
 *   rot = 0  tags in column order, rows in matrix order, Rpad = R rounded up to 4, one column order:
 *            read by the tensor-core products cbl_gemm_l8 / cbl_gemm_rows_multi (cbl_repack_l8);
 *   rot = 1  the batch-1 layout (cbl_repack_l8r): slot s of the stream at row position p holds chunk
 *            column (s + p / 4) mod 8, so that the lanes of a warp (4 rows each) read different columns at the same time;
 *            rows may be grouped by column order (row_index, seg_off), Rpad is a multiple of 32.
 * d = 8, bits = 12, G = 1.
 * replaces shapequant/kernels/proto_runs.py:322-336, 380-388 (pack_lane_major, make_tiles: load-time re-layout
 *          of the tags into the kernel's order, rows grouped by column order).
 * ------------------------------------------------------------------------------------------ */
#define CBL_L8_MAX_ORDERS 16
typedef struct cbl_l8 {
    int32_t R, C, books, ntile, Rpad;   /* ntile counts both books' tiles */
    int32_t rot;                        /* 0 or 1, see above */
    int32_t M;                          /* column orders (rot = 1; at most CBL_L8_MAX_ORDERS), else 1 */
    int32_t book_exp;                   /* rot = 1: cbl_book_norm_exp of frag (host-known, so that the kernel need not fetch it) */
    const void* words;                  /* uint32 [ntile][3][Rpad] */
    const void* frag;                   /* the 4096 x 8 book in tensor-core fragment order (cbl_repack_book) */
    const void* frag2;                  /* second book when books == 2 */
    const void* row_scale;              /* fp16 [R], by source row */
    const void* table;                  /* the book as stored, fp16 [4096, 8] (used by cbl_gemm_l8) */
    const void* table2;
    const int32_t* row_index;           /* rot = 1: source row of each row position, -1 = padding; NULL = identity */
    const int32_t* perms;               /* rot = 1, M > 1: int32 [M][C], the activation index of every stored column */
    int32_t seg_off[CBL_L8_MAX_ORDERS + 1];  /* rot = 1 (read on the HOST): positions [seg_off[m], seg_off[m+1]) hold the rows
                                           of column order m; multiples of 32, seg_off[0] = 0, seg_off[M] = Rpad */
    int32_t book_exp2;                  /* the same for frag2 when books == 2 */
} cbl_l8;

size_t cbl_l8_bytes(int32_t R, int32_t C, int32_t books);
int cbl_repack_l8(const cbl_packed* m, void* out, cbl_stream s);
/* The rot = 1 layout: out = cbl_l8r_bytes(Rpad, C, books) bytes; row_index as in the struct (device pointer or NULL). */
size_t cbl_l8r_bytes(int32_t Rpad, int32_t C, int32_t books);
int cbl_repack_l8r(const cbl_packed* m, const int32_t* row_index, int32_t Rpad, void* out, cbl_stream s);

/* A 4096 x 8 fp16 book re-ordered so that one 128-bit load per lane yields the mma.m16n8k8 A fragments
 * of two 16-codeword blocks, followed by the largest magnitude of the book as one float (64 KB + 16 B, done
 * once at load time; no counterpart in the reference, whose kernels copy the book to shared memory as stored:
 * shapequant/kernels/cuda_gemv.py:129-141). */
size_t cbl_book_frag_bytes(void);
int cbl_repack_book(const void* table, void* out, cbl_stream s);
/* floor(log2(largest Euclidean norm of a codeword)) of a book re-ordered by cbl_repack_book (clamped to -8 .. 24):
 * the exponent that scales the batch-1 kernel's tables.  Synchronises the stream (a load-time call). */
int cbl_book_norm_exp(const void* frag, int32_t* exp_out, cbl_stream s);

/* Batch-1 product by activation-side tables on the rot = 1 layout:
 *   y[r] = round_to(ydtype, row_scale[r] * sum_j <table[tag[r, j]], x[perms[m_r][8 j .. 8 j + 7]]>)   (perms = identity for M = 1)
 * Per tile the kernel computes T[e][c] = <table[e], x_chunk_c> once on the tensor cores (fp16 with a power-of-two
 * scale per tile, two alternating 64 KB tables in shared memory) and every weight chunk becomes one 2-byte
 * shared-memory read and an integer add (the entries are 16-bit integers with a power-of-two scale per tile).
 * Blocks that share rows store their fp32 partial sums into slots of the work space as {valid flag, value}
 * words; each block then sums a slice of the rows over the blocks in a fixed order (polling, with a bound, words
 * that have not landed yet), scales, rounds and writes y: one kernel per call, and repeated calls agree bit for bit.
 * Work space: cbl_gemv_l8_workspace_bytes(R) bytes, zero before the first call; every completed call leaves it
 * as it found it (slots zero).  Calls that share a work space must not overlap on the device.
 * Codeword magnitudes up to 2^13 are supported (larger ones may overflow the fp16 tables).
 * replaces shapequant/kernels/gemv.py:28-64, 142-162 (_gemv_kernel, PackedLinear.gemv) and
 *          shapequant/kernels/proto_runs.py:412-473, 505-571 (gemv_additive, gemv) for batch 1, including their
 *          input-side use of the column orders (proto_runs.py:500-502, prep_x) and the ordered split-K sum of
 *          shapequant/kernels/batched_runs.py:328-356. */
size_t cbl_gemv_l8_workspace_bytes(int32_t R);
int cbl_gemv_l8(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* workspace, cbl_stream s);

/* The work split cbl_gemv_l8_multi would use for a group on a device of max_blocks SMs, computed on the host
 * (no device needed; only R, C-derived ntile, M, Rpad and seg_off of the structs are read): every block takes
 * one rectangle of (row positions x tiles) of one matrix and column order, cut so that the slowest block is
 * as fast as possible under a cost model of table builds and lookups.  out: int32 [max_blocks][8] =
 * {matrix, column order, row part, tile splits of that part, first row position, rows, first tile, end tile}.
 * replaces the launch-shape heuristics of shapequant/kernels/proto_runs.py:505-571 (blocks per SM, split-K). */
int cbl_gemv_l8_plan(const cbl_l8* mats, int32_t n, int32_t max_blocks, int32_t* out, int32_t* nblocks);

/* Up to 4 matrices that read the same activation vector (q|k|v, gate|up) as ONE launch: the blocks are
 * shared out over all their (rows x tiles) rectangles, so launch and first-table latencies are paid once.
 * ys[i] receives matrix i's output; the work space holds the sum of cbl_gemv_l8_workspace_bytes(R_i) bytes
 * (zero before the first call).
 * replaces the merged q|k|v and gate|up launches of shapequant/kernels/decode_e2e.py:453-485
 *          (merge_runs) and the per-piece loop of shapequant/vllm_ext/core.py:376-384 (_small). */
int cbl_gemv_l8_multi(const cbl_l8* mats, int32_t n, const void* x, int xdtype, void* const* ys, int ydtype,
                      void* workspace, cbl_stream s);

/* Row-split (tensor-parallel o / down) batch-1 product fused with the sum over ranks, without a
 * collective library: each rank accumulates its chunk range locally, then one kernel per rank
 * exchanges "ready" words with its peers (bounded wait), reads every rank's partial sums through
 * peer pointers over NVLink, adds them in rank order (bit-identical on all ranks), scales, rounds and
 * writes the full y on every rank.  peer_ws[r] = rank r's work space (symmetric allocation mapped
 * into this process; cbl_gemv_l8_ar_workspace_bytes(R) bytes, zero before the first call, one work
 * space per matrix).  All ranks must issue the same sequence of calls; the call number is kept in the
 * work space by the kernels, so the launches can be captured in a CUDA graph and replayed.  At most
 * 8 ranks.  New with tensor parallelism (the reference has none); replaces product + NCCL all-reduce. */
size_t cbl_gemv_l8_ar_workspace_bytes(int32_t R);
int cbl_gemv_l8_ar(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, void* const* peer_ws, int32_t rank,
                   int32_t world, cbl_stream s);
/* CBL_ETIMEOUT if, since the last query, a peer's word did not arrive within the bounded wait of a
 * cbl_gemv_l8_ar call on this rank's work space (that call's output is invalid; the GPU context stays
 * usable and the next call on the same work space is correct again: every call overwrites the sums it
 * publishes).  Synchronises the stream and clears the word. */
int cbl_gemv_l8_ar_status(void* workspace, int32_t R, cbl_stream s);

/* The kernel's waits (on its staged copies, on the other blocks of a row part) are bounded; if one ever
 * expires the kernel sets a status word in the work space and leaves.  This call synchronises the stream and
 * returns CBL_OK or CBL_ETIMEOUT; after a time-out it also clears the work space (on that stream), so it
 * can be used again.  R is not used (kept for the signature of earlier versions).
 * (The reference's kernels spin without a bound, shapequant/kernels/proto_runs.py:234-243.) */
int cbl_gemv_l8_status(void* workspace, int32_t R, cbl_stream s);

/* The same batch-1 product for callers that cannot hand the library any device memory of their
 * own making (hosts that pre-partition the whole GPU into private pools, or plugin contracts that
 * forbid allocator calls while serving).  The product's work space lives in a fixed array compiled into
 * the library: 1 MB + 256 B of every GPU that loads the library stay reserved until the process exits, and the
 * launch uses at most 32 thread blocks so that their partial sums fit (slower than cbl_gemv_l8 on large
 * matrices, same results bit for bit when the work split is the same, within fp32 summation order otherwise).
 * Limit: cbl_gemv_l8_static_max_rows() = 65536 output rows (larger R: CBL_EUNSUPPORTED).
 * The call allocates and frees nothing.  Its first use on a device looks the array's device address
 * up (cudaGetSymbolAddress, under a lock), so make that first call before any stream capture.  All calls
 * share the one array, which keeps the last call's contents: a product that runs to its end clears every word
 * it used (the array starts zero), one that gave up leaves words behind until cbl_gemv_l8_static_status clears
 * them; two such products that overlap on the GPU (different streams, or a replayed graph beside a live call)
 * race on the array - serialise them.
 * cbl_gemv_l8_static_status(s): the bounded-wait status of such products on the current device since the last
 * query (CBL_OK or CBL_ETIMEOUT; synchronises the stream, after a time-out clears the array, allocates nothing).
 * No counterpart in the reference (its launchers allocate through torch / CuPy). */
int32_t cbl_gemv_l8_static_max_rows(void);
int cbl_gemv_l8_static(const cbl_l8* m, const void* x, int xdtype, void* y, int ydtype, cbl_stream s);
int cbl_gemv_l8_static_status(cbl_stream s);

/* ------------------------------------------------------------------------------------------
 * Prefill product on the column-tile layout (rot = 0): y[t*ldy + r] = round_to(ydtype, row_scale[r] *
 * sum_c W[r, c] * x[t*ldx + c]) for t < ntok.  W tiles are decoded into shared memory and multiplied
 * with tcgen05.mma (fp16 x fp16, fp32 accumulation in tensor memory); x is staged as fp16 with a
 * power-of-two scale per token in `stage` (cbl_gemm_stage_bytes).  `workspace`: at least 4 bytes,
 * zero; a nonzero word afterwards means a bounded device-side wait expired (output invalid).
 * A second summed book runs as a second pass over the activation k-blocks into the same accumulators.
 * replaces shapequant/kernels/runs_gemm.py:471-514 (gemm: fused dequant + GEMM with mma.sync) and the
 *          dequant + cuBLAS large-M path of shapequant/vllm_ext/core.py:386-420. */
size_t cbl_gemm_stage_bytes(int32_t ntok, int32_t C);
int cbl_gemm_l8(const cbl_l8* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                void* stage, void* workspace, cbl_stream s);

/* The same product computed by clusters of two thread blocks with tcgen05.mma.cta_group::2 (512-token x
 * 256-row tiles; each block decodes half of the weight tile).  Same arguments and results; measured
 * slower than cbl_gemm_l8 on B200 at present, kept as the two-SM variant of the design. */
int cbl_gemm_l8_2sm(const cbl_l8* m, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* y, int ydtype, int64_t ldy,
                    void* stage, void* workspace, cbl_stream s);

/* Up to cbl_gemm_rows_max_tokens() (32) tokens on the tensor cores with the WEIGHT ROWS as the M side of
 * tcgen05.mma: every block decodes 128 rows x its share of k into the swizzled A tile (each weight is
 * decoded once whatever the token count), the tokens are the N side (TMA).  Up to four matrices that share
 * the activations (q|k|v, gate|up; same C and book count) run as one launch; ys[i] receives
 * y_i[t * ldy + r].  Products with few row tiles are split along k, summed in `workspace`
 * (cbl_gemm_rows_workspace_bytes(sum of the matrices' padded rows) bytes, zero before the first call, left
 * zero; its last 16 bytes hold the status word) and finished by a second kernel.  x, stage as for cbl_gemm_l8.
 * One column order only (M = 1); one or two books.
 * replaces shapequant/kernels/batched_runs.py:745-771 (RunsBatch.run) for batches of 9..32 tokens. */
int32_t cbl_gemm_rows_max_tokens(void);
size_t cbl_gemm_rows_workspace_bytes(int32_t sum_rows_padded);
int cbl_gemm_rows_multi(const cbl_l8* mats, int32_t n, const void* x, int xdtype, int32_t ntok, int64_t ldx, void* const* ys, int ydtype,
                        int64_t ldy, void* stage, void* workspace, cbl_stream s);

/* ------------------------------------------------------------------------------------------
 * Activation-stationary layout ("x16") for 16..32 tokens on mma.sync: a warp keeps the activations of its
 * 128 input columns in registers (A fragments, tokens = M) and walks over the weight rows, 8 at a time
 * (N = 8): per 8 rows x 128 columns four 16-byte codeword reads per lane feed 8 (16 tokens) or 16 (32
 * tokens) MMAs, nothing else touches shared memory except the partial sums that the 16 warps of a block
 * (16 column ranges) add into a 64-row x 32-token tile.  Tags are stored per (column range, block of 64
 * rows) so that a lane reads its 32 tags (8 row tiles x 4 chunks) with three coalesced 16-byte loads.
 * d = 8, bits = 12, G = 1, M = 1; books = 2 stored as a second run.
 * replaces shapequant/kernels/batched_runs.py:745-771 (RunsBatch.run) for batches of 16..32 tokens.
 * ------------------------------------------------------------------------------------------ */
typedef struct cbl_x16 {
    int32_t R, C, books, nkr, nrb;     /* nkr = ceil(C / 128) column ranges, nrb = ceil(R / 64) row blocks */
    const void* words;                 /* uint4 [books][nkr][nrb][3][32] */
    const void* table;                 /* fp16 [4096, 8] */
    const void* table2;                /* fp16 [4096, 8] when books == 2 */
    const void* row_scale;             /* fp16 [R] */
} cbl_x16;

size_t cbl_x16_bytes(int32_t R, int32_t C, int32_t books);
int cbl_repack_x16(const cbl_packed* m, void* out, cbl_stream s);
/* y[t * ldy + r] = round(row_scale[r] * sum_c W[r, c] x[t, c]) for t < B <= 32.  xp: the activations staged by
 * cbl_prep_x (M = 1).  workspace: cbl_gemv_x16_workspace_bytes(R) bytes, zero before the first call, left zero
 * (fp32 sums of products whose columns are split over several blocks). */
size_t cbl_gemv_x16_workspace_bytes(int32_t R);
int cbl_gemv_x16(const cbl_x16* m, const void* xp, int32_t B, void* y, int ydtype, int64_t ldy, void* workspace, cbl_stream s);

/* Two-phase prefill for many tokens and for matrices with several column orders: decode the matrix ONCE
 * into a 16-bit scratch, then multiply with a TMA-fed tcgen05 GEMM (both operands by TMA, accumulators in
 * tensor memory).
 * Ordering: both kernels use programmatic dependent launch - cbl_decode_raw starts WRITING `out` while earlier work
 * of the stream may still be running (it waits for its predecessors only at its end, so that it runs beside the
 * previous GEMM), and cbl_gemm_dense lets the next kernel start early.  `out` must therefore not be read or
 * written by any earlier work of the stream that may still be in flight: a caller that decodes matrix after
 * matrix keeps TWO scratch buffers and alternates them (decode A, gemm A, decode B, gemm B, decode A, ...), as
 * DenseStack does; with a single scratch put an event or another kernel between a GEMM and the next decode.
 *   cbl_decode_raw: out fp16 [R, ld], ld = C rounded up to 8, = cbl_dense_scratch_bytes(R, C) bytes:
 *                   out[r, col] = fp16(A[tag]) or fp16(fp32(A[tag]) + fp32(B[tag2])), col the ORIGINAL column
 *                   (column orders undone), without the row scale.  d = 8, 12-bit tags, G = 1.
 *   cbl_gemm_dense: y[t, r] = round(row_scale[r] * sum_c out[r, c] * x[t, c]); x, y, stage, workspace as for
 *                   cbl_gemm_l8.  256-token x 256-row tiles.
 * replaces the dequant + cuBLAS large-M path of shapequant/vllm_ext/core.py:386-420 (_large) and the
 *          multi-token branch of shapequant/kernels/gemv.py:164-170 (dense() + F.linear). */
size_t cbl_dense_scratch_bytes(int32_t R, int32_t C);
int cbl_decode_raw(const cbl_packed* m, void* out, cbl_stream s);
/* The same for a column shard (tensor parallelism) of a matrix with several column orders: the shard's orders name
 * positions of the FULL activation vector, so a row of `out` is C_out >= m->C wide (ld = C_out rounded up to 8,
 * cbl_dense_scratch_bytes(R, C_out) bytes) and the shard's weights land at out[r, perms[row_mask[r]][c]]; every other
 * element must be ZERO on entry (the call writes only the shard's positions; every index in perms must be below
 * C_out).  The product is then cbl_gemm_dense over C_out columns against the full activations.
 * no counterpart in the reference (which refuses tensor parallelism, shapequant/vllm_ext/plugin.py:198-199). */
int cbl_decode_raw_wide(const cbl_packed* m, void* out, int32_t C_out, cbl_stream s);
int cbl_gemm_dense(const void* w16, int32_t R, int32_t C, const void* row_scale, const void* x, int xdtype, int32_t ntok, int64_t ldx,
                   void* y, int ydtype, int64_t ldy, void* stage, void* workspace, cbl_stream s);

/* ------------------------------------------------------------------------------------------------
 * Decode-step operators between the packed linears (Qwen2-style blocks).  `dtype` is the model's
 * 16-bit activation type (CBL_F16 or CBL_BF16) shared by every 16-bit pointer of a call; the residual
 * stream `h` is fp32.  Arithmetic follows the reference's batch-1 engine: activations are rounded to
 * the 16-bit type between operators, biases are added and silu * up is multiplied in that type, cos / sin
 * are rounded to it.  All calls enqueue on `s`, allocate nothing and do not synchronise.
 * replaces the CuPy kernels of shapequant/kernels/decode_e2e.py:63-309 (embed, addnorm_perm, rope_cache,
 * attn / attn_rope, silu_mul_perm), DenseLin.run (:329-341) and torch.argmax in DecodeEngine.step (:715),
 * and their batched forms in shapequant/kernels/qwen2_batch_kernels.py:37-88. */

/* h[b, :] = float(embed[tok[b] mod rows, :]) for b < B. */
int cbl_embed_rows(const void* embed, int dtype, int64_t rows, int32_t H, const int64_t* tok, int32_t B, float* h, cbl_stream s);

/* h[b] += add[b] (add may be NULL; row stride ld_add elements); x[b] = round(h[b] * rsqrt(mean(h[b]^2) + eps) * w).
 * x is [B, H] contiguous. */
int cbl_add_rmsnorm(float* h, const void* add, int64_t ld_add, const void* w, int dtype, float eps, int32_t B, int32_t H, void* x,
                    cbl_stream s);

/* Rotary embedding + cache write.  qkv [rows, ld] holds q heads | k heads | v heads per row; bias (NULL or
 * [(NH + 2 NKV) * HD]) is added first.  Row r belongs to sequence r at position pos[r] (decode, pos != NULL)
 * or to sequence seq0 at position pos0 + r (prefill, pos == NULL).  Writes the rotated queries to
 * q_out [rows, NH * HD], the rotated keys into the key cache [seq][NKV][max_len][HD] and the values into the
 * dimension-major value cache [seq][NKV][HD][max_len].
 * Rotation pairs element i with i + HD/2 (the Hugging Face convention). */
int cbl_rope_kv(const void* qkv, int dtype, int64_t ld, const void* bias, const int32_t* pos, int32_t pos0, int32_t seq0, int32_t rows,
                int32_t NH, int32_t NKV, int32_t HD, float theta, int32_t max_len, void* q_out, void* kc, void* vc, cbl_stream s);

/* Grouped-query attention of one new token per sequence over cache positions 0..pos[b] (the step's own
 * key / value already written by cbl_rope_kv), flash-decoding on tensor cores.  q, out: [B, NH * HD]; key cache
 * [B][NKV][max_len][HD], value cache dimension-major [B][NKV][HD][max_len]; HD = 128, NH / NKV <= 8, max_len a
 * multiple of 32, both caches zero (or finite) where nothing has been written yet.  pos[b] must lie in
 * [0, max_len); a position outside is clamped to the cache (the call reads no memory beyond it, the result is then
 * the attention over the whole cache) - cbl_rope_kv skips the cache write of such a row.  The positions of a sequence
 * are cut into `nsplit` slices (1..cbl_attn_decode_max_splits()) that run in parallel, four warps per slice;
 * `workspace` holds their partial results (cbl_attn_decode_workspace_bytes bytes; no initial contents required). */
size_t cbl_attn_decode_workspace_bytes(int32_t B, int32_t NH, int32_t nsplit);
int32_t cbl_attn_decode_max_splits(void);
int cbl_attn_decode(const void* q, const void* kc, const void* vc, const int32_t* pos, int dtype, int32_t B, int32_t NH, int32_t NKV,
                    int32_t HD, int32_t max_len, float scale, void* out, void* workspace, int32_t nsplit, cbl_stream s);

/* out[b, i] = round(round(silu(gate_up[b, i])) * gate_up[b, I + i]); gate_up [B, ld], out [B, I] contiguous. */
int cbl_silu_mul(const void* gate_up, int dtype, int64_t ld, int32_t B, int32_t I, void* out, cbl_stream s);

/* Dense 16-bit output head for small batches: logits[b, v] = <W[v, :], x[b, :]>, W [V, H] and x [B, H]
 * contiguous in `dtype`, fp32 accumulation, logits in `ldtype` (CBL_F32 / F16 / BF16) with row stride ldl.
 * B <= cbl_head_gemv_max_batch() (larger batches are a plain library GEMM), H a multiple of 8. */
int32_t cbl_head_gemv_max_batch(void);
int cbl_head_gemv(const void* W, const void* x, int dtype, int32_t B, int32_t V, int32_t H, void* logits, int ldtype, int64_t ldl,
                  cbl_stream s);

/* Batch-1 products followed by the step operator that consumes them, applied by one small kernel to the product's
 * finished fp32 sums (one launch less than product + operator on a stored vector, no round trip of the rounded vector
 * through memory).  Results equal the product followed by the separate
 * operator: the product is rounded to `dtype` first.  `workspace` as for cbl_gemv_l8_multi (the sum of
 * cbl_gemv_l8_workspace_bytes(R_i) bytes; zero before the first call, left zero).
 *   cbl_gemv_l8_silu_mul: gate_up[0..1] (equal row counts) -> out[i] = silu(gate.x)[i] * (up.x)[i]; y_gate / y_up
 *                         (NULL or [R] in `dtype`) also receive the two products, as the reference's launch leaves them
 *   cbl_gemv_l8_add_norm: h += W.x; xout = RMSNorm(h) * w   (R <= cbl_gemv_l8_add_norm_max_rows()); y (NULL or [R])
 *                         also receives the product
 *   cbl_gemv_l8_rope_kv:  qkv[0..2] = q, k, v projections -> bias, rotary at position pos[0], rotated
 *                         query to q_out [NH * HD], key / value into the caches of sequence 0
 * replaces the epilogue modes of the reference's run kernel (shapequant/kernels/proto_runs.py:223-287:
 * add + norm and silu * mul written by the last blocks) and its fused rope + attention prologue
 * (decode_e2e.py:200-250). */
int cbl_gemv_l8_silu_mul(const cbl_l8* gate_up, const void* x, int xdtype, void* out, void* y_gate, void* y_up, int dtype, void* workspace,
                         cbl_stream s);
int32_t cbl_gemv_l8_add_norm_max_rows(void);
int cbl_gemv_l8_add_norm(const cbl_l8* m, const void* x, int xdtype, float* h, const void* w, float eps, void* xout, void* y, int dtype,
                         void* workspace, cbl_stream s);
int cbl_gemv_l8_rope_kv(const cbl_l8* qkv, const void* x, int xdtype, const void* bias, const int32_t* pos, int32_t NH, int32_t NKV,
                        int32_t HD, float theta, int32_t max_len, void* q_out, void* kc, void* vc, int dtype, void* workspace,
                        cbl_stream s);

/* The reference's block-32 formats of the embedding and the output head (aux section of a packed file,
 * shapequant/packed.py:33-41):
 *   cbl_embed_rows_q4: 4-bit embedding, q uint8 [rows, H/2] (even column in the low nibble), scale fp16 [rows, H/32]:
 *                      h[b, i] = (nibble - 8) * scale[tok[b] mod rows, i / 32] (exact in fp32); H a multiple of 32.
 *                      replaces embed_q4 (shapequant/kernels/decode_e2e.py:74-85) and packed.q4_embed_rows (:151-155).
 *   cbl_head_gemv_q8:  8-bit head (Q8_0-like), q int8 [V, H], scale fp16 [V, H/32]:
 *                      logits[b, v] = sum over blocks of scale * <q, x[b]>, fp32 accumulation; x [B, H] contiguous in
 *                      `dtype`, B <= cbl_head_gemv_q8_max_batch(), `scratch` = cbl_head_q8_scratch_bytes(B, H) bytes.
 *                      replaces gemv_q8 (shapequant/kernels/proto_formats.py:413-462) behind Q8Lin.run
 *                      (decode_e2e.py:385-402). */
int cbl_embed_rows_q4(const void* q, const void* scale, int64_t rows, int32_t H, const int64_t* tok, int32_t B, float* h, cbl_stream s);
size_t cbl_head_q8_scratch_bytes(int32_t B, int32_t H);
int32_t cbl_head_gemv_q8_max_batch(void);
int cbl_head_gemv_q8(const void* q, const void* scale, const void* x, int dtype, int32_t B, int32_t V, int32_t H, void* logits, int ldtype,
                     int64_t ldl, void* scratch, cbl_stream s);

/* tok[b] = index of the first largest logit of row b; pos[b] += 1 when pos != NULL. */
int cbl_argmax(const void* logits, int ldtype, int64_t ldl, int32_t B, int32_t V, int64_t* tok, int32_t* pos, cbl_stream s);

#ifdef __cplusplus
}
#endif
#endif /* CBL_H */
