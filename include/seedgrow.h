/* seedgrow - C ABI of the B200 (sm_100a) re-quantise / residual / rANS library.
 *
 * This is the boundary a host program binds with ctypes / cgo / JNI in place of the reference's
 * kernel-launch protocol (CuPy RawModule: seedpack/gpuquant.py:206-219, 432-456; seedpack/qr.py:925-1090;
 * its C realisation for --cpu: seedpack/cpukernels.py:270-305).
 *
 * Conventions
 *   - every function returns an int status, SG_OK (0) on success; nothing throws, nothing traps;
 *   - pointers are DEVICE pointers unless the name starts with h_;
 *   - `device` is the CUDA ordinal that owns the buffers, `stream` a cudaStream_t (NULL = default
 *     stream); calls enqueue work and return without synchronising unless stated otherwise;
 *   - the caller owns every buffer; the library allocates no device memory, scratch space is passed in;
 *   - calls on different streams may run concurrently from different host threads.
 */
#ifndef SEEDGROW_H
#define SEEDGROW_H

#include <stddef.h>
#include <stdint.h>

#if defined(SG_BUILD) && defined(__GNUC__)
#define SG_API __attribute__((visibility("default")))
#else
#define SG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define SG_OK             0
#define SG_ERR_ARG        1   /* null pointer, negative size, unknown enum */
#define SG_ERR_TYPE       2   /* ggml type (or type/variant pair) not supported */
#define SG_ERR_SHAPE      3   /* row length not a multiple of the type's block size */
#define SG_ERR_ALIGN      4   /* an offset breaks the 16-byte alignment the vector loads need */
#define SG_ERR_IMATRIX    5   /* the type needs an importance matrix and none was given */
#define SG_ERR_SCRATCH    6   /* scratch buffer missing or too small */
#define SG_ERR_TABLES     7   /* IQ grids not installed on this device */
#define SG_ERR_CUDA       8   /* a CUDA runtime call failed; see sg_last_cuda_error() */
#define SG_ERR_OVERFLOW   9   /* an output slot was too small (rANS encode); retry with more */
#define SG_ERR_CORRUPT   10   /* a coded stream ended early or decoded out of range */
#define SG_ERR_LIMIT     11   /* a size exceeds a documented fixed maximum */

/* bits a kernel may OR into the device status word (read with sg_status_fetch) */
#define SG_ST_OFFGRID     1   /* an IQ quantiser ended on a point that is not in the grid map */
#define SG_ST_OVERFLOW    2   /* rANS encoder ran out of slot space */
#define SG_ST_CORRUPT     4   /* rANS decoder read past its stream */

/* source element types of sg_quantize_* */
#define SG_DT_BF16 0
#define SG_DT_F16  1
#define SG_DT_F32  2

/* ggml type ids handled (seedpack/requant.py:21-27) */
#define SG_Q4_0 2
#define SG_Q4_1 3
#define SG_Q5_0 6
#define SG_Q5_1 7
#define SG_Q8_0 8
#define SG_Q2_K 10
#define SG_Q3_K 11
#define SG_Q4_K 12
#define SG_Q5_K 13
#define SG_Q6_K 14
#define SG_IQ2_XXS 16
#define SG_IQ2_XS 17
#define SG_IQ3_XXS 18
#define SG_IQ1_S 19
#define SG_IQ4_NL 20
#define SG_IQ3_S 21
#define SG_IQ2_S 22
#define SG_IQ4_XS 23
#define SG_IQ1_M 29
#define SG_TQ1_0 34
#define SG_TQ2_0 35
#define SG_MXFP4 39
#define SG_NVFP4 40
#define SG_Q1_0 41
#define SG_Q2_0 42

/* One tensor of a quantise / dequantise launch.  All tensors of a launch live in the same source,
 * destination and importance buffers at these offsets.  Mirrors the per-row descriptor arrays
 * xoff / yoff / npr / woff of the reference launch (seedpack/gpuquant.py:432-456), one record per
 * tensor instead of one per row. */
typedef struct sg_tensor {
    int64_t x_off;     /* first weight, in ELEMENTS of the source buffer (multiple of 8)              */
    int64_t y_off;     /* first output byte in the destination buffer                                 */
    int64_t w_off;     /* first importance weight, in floats (multiple of 4); < 0 = no importance matrix */
    int64_t n_rows;    /* rows                                                                        */
    int64_t n_per_row; /* weights per row (multiple of the type's block size)                         */
} sg_tensor;

SG_API int sg_version(void);
SG_API const char *sg_status_string(int status);
/* text of the last CUDA error seen by the calling thread ("" if none) */
SG_API const char *sg_last_cuda_error(void);

/* weights per block and bytes per block of a ggml type (seedpack/requant.py:21-27); SG_ERR_TYPE if unknown */
SG_API int sg_type_info(int ggml_type, int *qk, int *block_bytes);
/* does quantize_<type> insist on an importance matrix (ggml-quants.c:3303, 3481, 4521, 4705, 5122) */
SG_API int sg_type_needs_imatrix(int ggml_type);

/* Device status word: kernels OR SG_ST_* bits into it instead of asserting.  Fetch synchronises the
 * stream, returns the bits in *h_bits and clears the word. */
SG_API int sg_status_fetch(int device, void *stream, int *h_bits);

/* ---- IQ lattice tables -----------------------------------------------------------------------------
 * Replaces GPUQuant._upload_tables / _build_tables (seedpack/gpuquant.py:311-353) and the host routines
 * iq2xs_init_impl / iq3xs_init_impl (ggml-quants.c:2854, 3704).  The maps and neighbour lists are built on
 * the host on first use (about a second) and copied to the device once; this is the only device
 * allocation the library makes (about 6 MB, kept until the process ends).  Synchronises `stream`.
 * Needed before quantising IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M. */
SG_API int sg_tables_install(int device, void *stream);
/* host view of a built table, for tests: which = 0 IQ2_XXS, 1 IQ2_XS, 2 IQ1_S/M, 3 IQ2_S, 4 IQ3_XXS, 5 IQ3_S;
 * what = 0 grid (uint64 / uint32 per point), 1 map (int32), 2 neighbour lists (uint16) */
SG_API int sg_tables_host(int which, int what, const void **h_ptr, size_t *h_bytes);

/* ---- quantisers -------------------------------------------------------------------------------
 * Replaces k_quantize_<type>[_v1] (seedpack/gpuquant.py:206-211), i.e. llama.cpp's
 * quantize_<type>(row, dst, 1, n_per_row, imatrix) per row (ggml-quants.c:1212 ... 5283), byte for byte.
 * `variant` 0 = current arithmetic, 1 = older IQ1_M split search (seedpack/gpuquant.py:182-185).
 *
 * Scratch: the legacy importance paths (Q4_0, Q4_1, Q5_0, Q5_1 with an importance matrix) need one
 * float per row for the row-wide mean square (ggml-quants.c:2082-2084); sg_quantize_scratch_bytes()
 * gives the size for a launch, 0 when none is needed.  The buffer is written by the call and may be
 * reused by the next call on the same stream. */
SG_API size_t sg_quantize_scratch_bytes(int ggml_type, const sg_tensor *h_tensors, int n_tensors);
SG_API int sg_quantize_tensors(int device, void *stream, int ggml_type, int variant,
                        const void *x, int x_dtype, void *y, const float *w,
                        const sg_tensor *h_tensors, int n_tensors,
                        void *scratch, size_t scratch_bytes);

/* Dequantise n_weights weights of ggml type T (a multiple of its block size) to float32 with the arithmetic of
 * dequantize_row_<type>; replaces k_dq_<type> (seedpack/gpuquant.py:215-219).  Lattice types need sg_tables_install. */
SG_API int sg_dequantize(int device, void *stream, int T, const unsigned char *y, float *x, long long n_weights);
/* BF16 / F16 / F32 (SG_DT_*) to any of the three; to BF16 rounds to nearest even on the bits, to F16 IEEE round to
 * nearest; replaces M28RepoGPU._float_dev (seedpack/repo3.py:673-689) */
SG_API int sg_convert_float(int device, void *stream, const void *src, int src_dtype, void *dst, int dst_dtype,
                            long long n);

/* ---- per-block residual ------------------------------------------------------------------------------
 * Replaces the host-side NumPy helpers _xor_async / _diff_async / _count_diff / _xor3 (seedpack/repo3.py:456-510),
 * which need a device-to-host copy of every prediction first.
 *
 * sg_residual_xor: out = a ^ b ^ c over nbytes (b and c may be NULL; out may be NULL when only the count is
 * wanted, and may alias a).  *d_nonzero (device, caller-zeroed, accumulated with atomics) += non-zero bytes of
 * the result: with b this is _count_diff(a, b); 0 means "prediction exact".  Any alignment is accepted; 16-byte
 * aligned pointers take the vector path. */
SG_API int sg_residual_xor(int device, void *stream, const void *a, const void *b, const void *c, void *out,
                           size_t nbytes, unsigned long long *d_nonzero);
/* Block-wise comparison of a stored tensor with its prediction (same(), seedpack/qr.py:114-117): ne_flags[i]
 * (optional) = 1 where block i differs, *d_differ += number of differing blocks.  block_bytes must be even. */
SG_API int sg_residual_blocks(int device, void *stream, const void *file, const void *pred, int block_bytes,
                              long long n_blocks, unsigned char *ne_flags, unsigned long long *d_differ);

/* ---- segment-parallel rANS over a symbol stream ------------------------------------------------------
 * The coder of the reference's residual and base codecs (PUT / GET, seedpack/qr.py:651-663; seedpack/rans.py:54-105
 * with PROB_BITS = pb): 32-bit state, byte renormalisation, RANS_L = 2^23, static tables whose frequencies sum
 * to 2^pb.  Stream model: nsym byte symbols in blocks of block_len (multiple of 16); block b uses context table
 * block_tab[b]; segments of seg_len symbols (multiple of block_len) are independent streams.  A segment's bytes
 * are its final state, big endian, then the renormalisation bytes in decode order - the layout of the `s` part of
 * a QR batch (seedpack/qr.py:1058-1061).
 *
 * sg_rans_hist    counts[tab * 256 + sym] += occurrences (caller zeroes counts)          (qr_hist's hadd, qr.py:380-383)
 * sg_rans_tables  frequencies [ntab][256] (each used row summing to 2^pb) -> encoder entries enc_tab
 *                 (8 bytes per (table, symbol): reciprocal, freq | cum << 16) and, if lut != NULL, the decoder's
 *                 symbol-per-slot table [ntab << pb]                                     (cum_of gpu2.py:483-486, build_lut qr.py:889-895)
 *                 For pb = 15 `lut` is the R2 decoder's compact table instead, 1280 bytes per table [ntab * 1280]:
 *                 256 coarse entries (entry b = the symbol whose range holds slot 128 * b) and the 256 symbols'
 *                 freq | cum << 16 words; the decoder walks on from the coarse entry (32 KiB of slots per table would
 *                 not stay in the SM's cache, this does).
 * sg_rans_encode  every segment into its private slot of `cap` bytes (multiple of 16, >= 128), written from the
 *                 slot's end downwards; out_len[s] = bytes used, 0xffffffff = slot too small   (qr_enc's framing, qr.py:712-758)
 * sg_scan_gather  off[0..nseg] = exclusive prefix sum of out_len (off[nseg] = total), then the segments' bytes
 *                 copied to dst + off[s]; an overflowed segment sets SG_ST_OVERFLOW      (cumsum + gather, qr.py:1054-1056, 880-887)
 * sg_rans_decode  inverse of encode; reads of segment s stay inside [off[s], off[s+1]) and a segment that does
 *                 not end in the initial state sets SG_ST_CORRUPT (the reference reads unchecked, qr.py:662).
 *                 `in` must be 16-byte aligned and readable up to the next multiple of 16 past off[nseg].
 *                 ntab = number of tables in enc_tab / lut: with it the decoder keeps symbol 0's frequencies and the
 *                 other slots' entries in shared memory (0: not given, every symbol costs two dependent global loads). */
SG_API int sg_rans_hist(int device, void *stream, const unsigned char *sym, const unsigned short *block_tab,
                        int block_len, long long nsym, unsigned *counts);
SG_API int sg_rans_tables(int device, void *stream, const unsigned short *freq, int ntab, int pb, void *enc_tab,
                          unsigned char *lut);
SG_API int sg_rans_encode(int device, void *stream, const unsigned char *sym, const unsigned short *block_tab,
                          int block_len, long long nsym, int seg_len, int pb, const void *enc_tab,
                          unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_scan_gather(int device, void *stream, const unsigned char *slots, size_t cap, const unsigned *out_len,
                          int nseg, unsigned char *dst, unsigned long long dst_cap, unsigned long long *off);
SG_API int sg_rans_decode(int device, void *stream, const unsigned char *in, const unsigned long long *off,
                          const unsigned short *block_tab, int block_len, long long nsym, int seg_len, int pb,
                          const void *enc_tab, const unsigned char *lut, int ntab, unsigned char *sym_out);

/* ---- QR: quantiser-aware residual coder ---------------------------------------------------------------
 * Replaces qr_hist / qr_enc / qr_dec (seedpack/qr.py:674-807) for the scalar-code types (2 3 6 7 8 10 11 12 13 14
 * 20 23 42) and the lattice types (16 17 18 19 21 22 29; these need sg_tables_install first and use the importance
 * vector imx + TM.imx_off of each tensor, imx_off < 0 = none; imx may be NULL when no tensor has one).  A batch = tensors of one ggml type T laid back to back as blocks:
 *   F stored blocks, P predicted blocks (both nblocks * block_bytes), ne[b] = 1 where block b differs from its
 *   prediction (from sg_residual_blocks), seed = base weights buffer (per tensor: byte offset + type in TM),
 *   tm / sg = per-tensor and per-segment records with the reference's layouts
 *     TM { int64 blk0, seed_off; int32 seed_type, cols; int64 imx_off }   (qr.py:898)
 *     SG { int32 t, nb; int64 b0 }                                        (qr.py:900)
 *   seed types: 30 BF16, 0 F32, 1 F16, 98 none (per-column RMS floats), 99 explicit (x, h) float pairs, or one of the
 *   scalar-code quant types (the seed buffer then holds that type's blocks: value = dequantised weight, uncertainty =
 *   half a code step; qr.py:331-344).
 * Context tables are addressed by their raw id (0..293, qr.py:50-53): counts is [294 * 256], enc_tab / lut come from
 * sg_rans_tables on the full 294-row frequency array (unused rows zero), pb = 12.  mv = model version (1 or 2,
 * qr.py:54).  Streams, slots, out_len and offsets are those of sg_rans_encode / sg_scan_gather / sg_rans_decode.
 * sg_qr_decode writes every block of F (equal blocks are copied from P). */
SG_API int sg_qr_hist(int device, void *stream, int T, const unsigned char *F, const unsigned char *P,
                      const unsigned char *ne, const unsigned char *seed, const void *tm, const void *sg, int nseg,
                      const float *imx, unsigned *counts, int mv);
SG_API int sg_qr_encode(int device, void *stream, int T, const unsigned char *F, const unsigned char *P,
                        const unsigned char *ne, const unsigned char *seed, const void *tm, const void *sg, int nseg,
                        const float *imx, const void *enc_tab, unsigned char *slots, size_t cap, unsigned *out_len,
                        int mv);
/* Encoding in two steps, for throughput: the model of a block (fields, predictions, contexts, lattice ranks) does not
 * depend on the coder's state, so sg_qr_stage runs it once with one lane per BLOCK and writes every block's
 * (table, symbol) pairs into `stage` (sg_qr_stage_bytes(T, nblocks) bytes, 16-byte aligned, owned by the caller);
 * sg_qr_stage_hist counts the pairs into counts[294 * 256] (add to what is there), and sg_qr_stage_encode walks
 * them with one rANS lane per segment.  Same bytes out as sg_qr_hist + sg_qr_encode, which run the model twice
 * on one lane per segment.  nblocks = blocks of the whole batch.  No counterpart in the reference, which has the
 * single-pass kernels only (seedpack/qr.py:674-758). */
SG_API size_t sg_qr_stage_bytes(int T, long long nblocks);
SG_API int sg_qr_stage(int device, void *stream, int T, const unsigned char *F, const unsigned char *P,
                       const unsigned char *ne, const unsigned char *seed, const void *tm, const void *sg, int nseg,
                       const float *imx, int mv, long long nblocks, void *stage, size_t stage_bytes);
SG_API int sg_qr_stage_hist(int device, void *stream, int T, long long nblocks, const void *stage, unsigned *counts);
SG_API int sg_qr_stage_encode(int device, void *stream, int T, long long nblocks, const void *stage, const void *sg,
                              int nseg, const void *enc_tab, unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_qr_decode(int device, void *stream, int T, const unsigned char *in, const unsigned long long *off,
                        const unsigned char *P, const unsigned char *seed, const void *tm, const void *sg, int nseg,
                        const float *imx, const void *enc_tab, const unsigned char *lut, unsigned char *F, int mv);

/* ---- R2: BF16 base-model codec and its order-fixed statistics ------------------------------------------------
 * Replaces v2_hist / v2_enc / v2_dec / row_hash (seedpack/bf16v2.py:63-155) and the statistics of BF16v2._stats
 * (seedpack/bf16v2.py:225-244) built on detmath (seedpack/detmath.py:67-106).  15 probability bits, segments of 16384
 * weights, symbols per weight in decode order: exponent, mantissa, sign.  Records keep the reference's layouts:
 *   TB { int64 doff; int32 rowlen, rowbase, colbase, tab, rmap, pad }   one per tensor of the launch (bf16v2.py:158)
 *   SG { int32 t, n; int64 i0 }                                         one per segment                (bf16v2.py:159)
 * dev = buffer holding the tensors (TB.doff = byte offset), rfi / cfi / scl = side information (int16 per row, int16 and
 * int8 per column), rowmap = compact-to-original row numbers of tensors with duplicate rows removed (TB.rmap >= 0).
 * Tables are addressed by raw id (role * 656 + context): counts has nroles * 656 * 256 entries; enc_tab / lut come
 * from sg_rans_tables(..., pb = 15).  sg_r2_decode takes the first and one-past-last stream byte of every segment.
 * sg_r2_stats writes rfi[nrows], cfi[rowlen], scl[rowlen] of one tensor; scratch from sg_r2_stats_scratch_bytes. */
SG_API int sg_r2_hist(int device, void *stream, const unsigned char *dev, const void *tb, const void *sg, int nseg,
                      const short *rfi, const short *cfi, const signed char *scl, const int *rowmap, unsigned *counts);
SG_API int sg_r2_encode(int device, void *stream, const unsigned char *dev, const void *tb, const void *sg, int nseg,
                        const short *rfi, const short *cfi, const signed char *scl, const int *rowmap,
                        const void *enc_tab, unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_r2_decode(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                        const unsigned long long *in_end, unsigned char *dev, const void *tb, const void *sg, int nseg,
                        const short *rfi, const short *cfi, const signed char *scl, const int *rowmap,
                        const void *enc_tab, const unsigned char *lut);
/* 64-bit fingerprint of every row of a (nrows, rowlen) uint16 matrix (row_hash, bf16v2.py:148-155) */
SG_API int sg_row_hash(int device, void *stream, const void *w, int nrows, int rowlen, unsigned long long *h);
/* w[pairs[2p]] = w[pairs[2p + 1]] for rows of rowlen uint16: duplicate rows restored after decoding (bf16v2.py:475-480) */
SG_API int sg_copy_rows(int device, void *stream, void *w, int rowlen, const long long *pairs, int npairs);
SG_API size_t sg_r2_stats_scratch_bytes(int nrows, int rowlen);
SG_API int sg_r2_stats(int device, void *stream, const void *w, int nrows, int rowlen, short *rfi, short *cfi,
                       signed char *scl, void *scratch, size_t scratch_bytes);
/* detmath (seedpack/detmath.py:67-106, 178-215): float64 log2 / exp2 from IEEE basic operations; sums (of squares)
 * along rows / down columns of a float32 matrix in index order; mask (optional) leaves rows out of the column sums */
SG_API int sg_dm_log2(int device, void *stream, const double *x, long long n, double *y);
SG_API int sg_dm_exp2(int device, void *stream, const double *x, long long n, double *y);
SG_API int sg_dm_rows(int device, void *stream, const float *x, long long nr, long long nc, int square, double *out);
SG_API int sg_dm_cols(int device, void *stream, const float *x, long long nr, long long nc, int square,
                      const unsigned char *mask, double *out);

/* Helpers of the QR coder for tensors coded without a BF16 seed (seedpack/qr.py:811-878: block_fields,
 * blocks_from_fields, intervals, weq, grid_h): the blocks' scale fields as integers (nfield(T) per block, the same
 * field vector the coder works on) and blocks rebuilt from fields with all-zero codes; per weight the interval of
 * original values that rounds to its code, whether code and sub-block integer scale equal another tensor's, and - for
 * the lattice types - half the step between the lattice's levels.  Scalar-code types 2 3 6 7 8 10 11 12 13 14 20 23
 * 42, lattice types 16 17 18 19 21 22 29 where stated; SG_ERR_TYPE otherwise. */
SG_API int sg_qr_block_fields(int device, void *stream, int T, const unsigned char *F, long long nblocks, int *out);
SG_API int sg_qr_blocks_from_fields(int device, void *stream, int T, const int *fields, int nblocks, unsigned char *out);
SG_API int sg_qr_intervals(int device, void *stream, int T, const unsigned char *F, long long nweights, float *lo, float *hi);
SG_API int sg_qr_weight_equal(int device, void *stream, int T, const unsigned char *F, const unsigned char *P,
                              long long nweights, unsigned char *out);
SG_API int sg_qr_grid_half_step(int device, void *stream, int T, const unsigned char *F, long long nweights, float *h);

/* ---- M21: Q8_0 GGUFs that no base predicts (the seed of a repository without its BF16 model) ----------------------------
 * Replaces hist_a / enc_a / dec_a / hist_b / enc_b / dec_b (seedpack/gpu2.py:100-262) and predict / predict_multi /
 * hist_c / enc_c / dec_c (seedpack/gpu3.py:90-232); arguments in the reference's order and meaning.  blocks = Q8_0 blocks
 * of all tensors back to back, pos[b] = index of block b's largest magnitude, skip[b] = bit 0: not coded, bit 1: its 31
 * codes belong to phase C, bit 2: so do position and largest code; meta = per tensor { int32 first, nblocks, nb_row, grp,
 * colbase, rowbase, off, qset } (gpu2.py:56).  flags = the reference module's compile-time switches: bit 0 SIGN, bit 1
 * RANK, bit 2 HICF, bit 3 PREDA; seg = blocks per segment (SEGA / SEGB).  Tables by raw id (counts / enc_tab / lut from
 * sg_rans_tables with pb = 12 over the id space of the call); encoders write segment s at the end of slot s of `cap` bytes
 * (a multiple of 16) and out_len[s] = its bytes, 0xffffffff if the slot was too small (the reference does not look);
 * decoders take the first and one-past-last stream byte of every segment and report damage through SG_ST_CORRUPT.
 * sg_m21_decode_c decodes segments seg0 .. nseg - 1 (one wave of the format per call), one segment per CTA with the
 * tables of its 64 (88 with PREDA) contexts rebuilt in shared memory from enc_tab; its `lut` is not read and may be NULL. */
SG_API int sg_m21_hist_a(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                         const unsigned char *skip, const void *meta, int ntens, int nblocks, const unsigned char *bcf,
                         const unsigned char *spread, const unsigned char *perm, const unsigned char *rankof,
                         const unsigned char *scls, int flags, int seg, unsigned *counts);
SG_API int sg_m21_encode_a(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                           const unsigned char *skip, const void *meta, int ntens, int nblocks, const unsigned char *bcf,
                           const unsigned char *spread, const unsigned char *perm, const unsigned char *rankof,
                           const unsigned char *scls, int flags, int seg, const void *enc_tab, unsigned char *slots,
                           size_t cap, unsigned *out_len);
SG_API int sg_m21_decode_a(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                           const unsigned long long *in_end, const unsigned char *skip, const void *meta, int ntens,
                           int nblocks, const unsigned char *bcf, const unsigned char *spread, const unsigned char *perm,
                           const unsigned char *rankof, const unsigned char *scls, int flags, int seg,
                           const void *enc_tab, const unsigned char *lut, unsigned char *blocks, unsigned char *pos);
SG_API int sg_m21_hist_b(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                         const unsigned char *skip, const void *meta, int ntens, int nblocks, const short *cfi,
                         const unsigned char *scls, const int *row_m, int qbase, int G, int flags, int seg,
                         unsigned *counts);
SG_API int sg_m21_encode_b(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                           const unsigned char *skip, const void *meta, int ntens, int nblocks, const short *cfi,
                           const unsigned char *scls, const int *row_m, int qbase, int flags, int seg,
                           const void *enc_tab, unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_m21_decode_b(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                           const unsigned long long *in_end, const unsigned char *skip, const void *meta, int ntens,
                           int nblocks, const short *cfi, const unsigned char *scls, const int *row_m, int qbase,
                           int flags, int seg, const void *enc_tab, const unsigned char *lut, unsigned char *blocks,
                           const unsigned char *pos);
SG_API int sg_m21_predict(int device, void *stream, const unsigned char *blocks, int first, int nbr, int C,
                          const int *rows, int nrw, const int *par, const float *coef, int K, const float *mu,
                          signed char *pint);
SG_API int sg_m21_predict_multi(int device, void *stream, const unsigned char *blocks, const int *ent_slot,
                                const int *ent_row, int nent, int CMAX, const int *s_first, const int *s_nbr,
                                const long long *s_rbase, const long long *s_pbase, const int *s_mubase,
                                const int *par, const float *coef, int K, const float *mu, signed char *pint);
SG_API int sg_m21_hist_c(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                         const unsigned char *skip, const void *meta, const int *seg_t, const int *seg_r0,
                         const int *seg_nr, const int *seg_slot, int nseg, const short *cfi, const int *row_m,
                         const signed char *fbin, const long long *rbase, const signed char *pint,
                         const long long *pbase, int flags, unsigned *counts);
SG_API int sg_m21_encode_c(int device, void *stream, const unsigned char *blocks, const unsigned char *pos,
                           const unsigned char *skip, const void *meta, const int *seg_t, const int *seg_r0,
                           const int *seg_nr, const int *seg_slot, int nseg, const short *cfi, const int *row_m,
                           const signed char *fbin, const long long *rbase, const signed char *pint,
                           const long long *pbase, int flags, const void *enc_tab, unsigned char *slots, size_t cap,
                           unsigned *out_len);
SG_API int sg_m21_decode_c(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                           const unsigned long long *in_end, int seg0, unsigned char *pos, const unsigned char *skip,
                           const void *meta, const int *seg_t, const int *seg_r0, const int *seg_nr,
                           const int *seg_slot, int nseg, const short *cfi, const int *row_m, const signed char *fbin,
                           const long long *rbase, const signed char *pint, const long long *pbase, int flags,
                           const void *enc_tab, const unsigned char *lut, unsigned char *blocks);

/* M30, sibling quantisations without the model (seedpack/siblings.py:51-77: half_step, est_add, est_seed): element-wise
 * over n weights.  half_step: h = half the width of [lo, hi] (from sg_qr_intervals), the distance to the finite side when
 * one is infinite, -1 when both are.  est_add: a version (x, h) into the running sums ws += 1 / max(h^2, 1e-30),
 * wx += x * that (h < 0: skipped).  est_seed: the explicit QR seed, out[2i] = wx / ws, out[2i + 1] = 1 / sqrt(ws); where
 * ws is 0: (x0[i], 0). */
SG_API int sg_sib_half_step(int device, void *stream, const float *x, const float *lo, const float *hi, long long n, float *h);
SG_API int sg_sib_est_add(int device, void *stream, const float *x, const float *h, long long n, float *ws, float *wx);
SG_API int sg_sib_est_seed(int device, void *stream, const float *ws, const float *wx, const float *x0, long long n, float *out);

/* ---- M24: the earlier BF16 base codec (archives packed with --method m28) ---------------------------------------------
 * Replaces bf_hist / bf_enc / bf_dec (seedpack/gpu_bf16.py:63-137): 12 probability bits, 160 tables per tensor (128
 * exponent, 16 mantissa, 16 sign), quarter-octave side information.  file = the whole GGUF on the device; records
 *   TB { int64 off; int32 rowlen, rowbase, colbase, tab }   (gpu_bf16.py:283), SG { int32 t, n; int64 i0 }   (:284).
 * counts / enc_tab / lut cover ntensors * 160 tables addressed by raw id (sg_rans_tables with pb = 12); slots, out_len,
 * in_off / in_end as for the R2 entry points. */
SG_API int sg_m24_hist(int device, void *stream, const unsigned char *file, const void *tb, const void *sg, int nseg,
                       const short *rfi, const short *cfi, const signed char *scl, unsigned *counts);
SG_API int sg_m24_encode(int device, void *stream, const unsigned char *file, const void *tb, const void *sg, int nseg,
                         const short *rfi, const short *cfi, const signed char *scl, const void *enc_tab,
                         unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_m24_decode(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                         const unsigned long long *in_end, unsigned char *file, const void *tb, const void *sg, int nseg,
                         const short *rfi, const short *cfi, const signed char *scl, const void *enc_tab,
                         const unsigned char *lut);

/* ---- M6: the first GPU codec, Q8_0 files without a base ------------------------------------------------------------------
 * Replaces hist / encode / decode of seedpack/gpu_codec.py:73-159.  blocks = the file's Q8_0 blocks back to back (34 bytes
 * each), pos[b] = index of block b's largest magnitude, meta = per tensor { int32 first, nblocks, nb_row, grp, colbase,
 * med } (gpu_codec.py:182-183), tfirst[t] = first block of tensor t, colmap = a class byte per column; segments of 512
 * blocks; 770 tables per tensor group addressed by raw id (counts / enc_tab / lut cover ngroups * 770, sg_rans_tables with
 * pb = 12, the frequency array as the reference holds it: one row per table, unused rows zero); the encoder's slot must
 * hold a segment (the reference uses cap = 512 * 34 * 2 + 16, rounded up to 16 here by the caller). */
SG_API int sg_m6_hist(int device, void *stream, const unsigned char *blocks, const unsigned char *pos, const void *meta,
                      const int *tfirst, int ntens, const unsigned char *colmap, int nblocks, unsigned *counts);
SG_API int sg_m6_encode(int device, void *stream, const unsigned char *blocks, const unsigned char *pos, const void *meta,
                        const int *tfirst, int ntens, const unsigned char *colmap, int nblocks, const void *enc_tab,
                        unsigned char *slots, size_t cap, unsigned *out_len);
SG_API int sg_m6_decode(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                        const unsigned long long *in_end, const void *meta, const int *tfirst, int ntens,
                        const unsigned char *colmap, int nblocks, const void *enc_tab, const unsigned char *lut,
                        unsigned char *blocks);

/* ---- the scalar stream coder of the first codec generations -------------------------------------------------------------
 * Replaces _encode / _decode of seedpack/rans.py:54-105 (one rANS state per stream, 14 probability bits, a table number
 * per symbol from the caller), as M22's BF16 codec uses them (seedpack/bf16codec.py:56-58, 88-92).  A launch codes
 * nchain streams that share tables, one lane each: stream c covers the symbols [sym_off[c], sym_off[c + 1]) of sym and
 * ctx (ctx elements of 1, 2 or 4 bytes, unsigned; a value >= ntab marks the stream).  Encode writes stream c at the END
 * of slots[slot_off[c] .. slot_off[c + 1]) (16-byte aligned offsets; the reference sizes a slot 2 * symbols + 16) and
 * out_len[c] = its bytes, 0xffffffff when the slot was too small, 0xfffffffe for a symbol without frequency.  Decode
 * reads stream c from in[in_off[c] .. in_end[c]) and, when `used` is given, stores how many bytes it consumed (what
 * rans.py's _decode returns); enc_tab / lut from sg_rans_tables with pb = 14. */
SG_API int sg_rans_chain_encode(int device, void *stream, const unsigned char *sym, const void *ctx, int ctx_bytes,
                                const unsigned long long *sym_off, int nchain, int ntab, const void *enc_tab,
                                unsigned char *slots, const unsigned long long *slot_off, unsigned long long *out_len);
SG_API int sg_rans_chain_decode(int device, void *stream, const unsigned char *in, const unsigned long long *in_off,
                                const unsigned long long *in_end, const void *ctx, int ctx_bytes,
                                const unsigned long long *sym_off, int nchain, int ntab, const void *enc_tab,
                                const unsigned char *lut, unsigned char *sym_out, unsigned long long *used);

/* The remaining detmath kernels (seedpack/detmath.py:86-93, 109-153: dm_rows_d, dm_gram, dm_bdot, dm_solve), which the
 * importance fit uses (seedpack/imxfit.py:36-75): sums (of squares) along the rows of a float64 matrix; batched
 * X[c] X[c]^T (X: nb x k x d float32 -> nb x k x k float32) and X[c] y[c] (-> nb x k) with float64 sums in index order;
 * batched systems A[c] x = b[c] with k <= 16 unknowns (SG_ERR_LIMIT beyond) by Gaussian elimination with partial
 * pivoting in float64. */
SG_API int sg_dm_rows_f64(int device, void *stream, const double *x, long long nr, long long nc, int square, double *out);
SG_API int sg_dm_gram(int device, void *stream, const float *X, long long nb, int k, long long d, float *out);
SG_API int sg_dm_bdot(int device, void *stream, const float *X, const float *y, long long nb, int k, long long d, float *out);
SG_API int sg_dm_solve(int device, void *stream, const float *A, const float *b, long long nb, int k, float *x);

/* Diagnostic: out[i] = nearest_int(x[i]), the magic-number rounding every quantiser uses (ggml-quants.c:621-626), so that
 * the device form can be swept over its whole input range on its own (tests/test_helpers_gpu.py).  The conversions
 * f32 -> f16 / f16 -> f32 (ggml-impl.h:396-443) are swept through sg_convert_float. */
SG_API int sg_selftest_nearest_int(int device, void *stream, const float *x, int *out, long long n);

/* Allocation-free variant for hosts that cannot tolerate (or cannot supply memory for) a device allocation while
 * they run - a packer that has split the measured free device memory into fixed windows, or a pipeline whose
 * other streams must not be stalled by cudaMalloc's device-wide synchronisation.  It has no counterpart in the
 * reference, whose kernels take every buffer from the caller's CuPy pool.
 *
 * Same result as sg_quantize_tensors for Q4_0, Q4_1, Q5_0, Q5_1 WITH an importance matrix (every tensor needs
 * w_off >= 0; other types and matrix-free tensors need no scratch, use sg_quantize_tensors), but the per-row
 * scratch is a fixed 256 KiB array inside the library, present on every GPU that loads it until the process exits.
 * Limits and rules:
 *   - at most 65536 rows per call over all tensors, else SG_ERR_LIMIT (split the launch);
 *   - the first call on a device looks up the array's device address; make that first call outside any stream
 *     capture;
 *   - all calls share the one array (it is fully rewritten by each call before it is read, nothing needs
 *     clearing), so two calls whose kernels may overlap on the GPU - different streams, or different threads -
 *     race on it: keep calls to this entry point on one stream per device.
 * Calls cudaMalloc / cudaFree never; returns the same status codes as sg_quantize_tensors. */
SG_API int sg_quantize_legacy_imx_static(int device, void *stream, int ggml_type, const void *x, int x_dtype,
                                         void *y, const float *w, const sg_tensor *h_tensors, int n_tensors);

#ifdef __cplusplus
}
#endif
#endif /* SEEDGROW_H */
