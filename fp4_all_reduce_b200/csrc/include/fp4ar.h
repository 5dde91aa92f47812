/* fp4ar: NVFP4-transport tensor-parallel AllReduce for B200 (sm_100a) -- public C interface.
 *
 * One context per tensor-parallel group member.  A context owns nothing but a few hundred bytes of
 * device state; the receive window (peer-mapped memory, one per rank, every rank able to store into
 * every other rank's window) is allocated by the caller and handed in as an array of device pointers.
 * Every launch is asynchronous on the given stream, takes no host-side per-call state (the call index
 * lives on the device) and can therefore be captured in a CUDA graph.
 *
 * Counterpart in the reference project: include/fp4ar_api.h:10-53 (Fp4ArCtx / Fp4ArArgs / Fp4ArVariant)
 * and the free functions lnorm_window_bytes / lnorm_init / lnorm_launch / lnorm_fini in
 * kernels/fused_norm/lnorm.cu:726-770.  Differences: one entry point covers every tensor-parallel degree
 * (1, 2, 4, 8), both algorithms, the three input kinds and the four epilogues; waits are bounded and
 * report through fp4ar_status(); the window is half the size because receive slots are re-armed by
 * their consumer inside the same call.
 */
#ifndef FP4AR_H_
#define FP4AR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FP4AR_MAX_RANKS 8
#define FP4AR_HIDDEN 6144
#define FP4AR_QROW_BYTES 3456   /* NVFP4 row: 3072 value bytes then 384 scale bytes */
#define FP4AR_MXROW_BYTES 6336  /* MXFP8 row: 6144 value bytes then 192 UE8M0 scale bytes */
#define FP4AR_REC_STRIDE 3584   /* pitch of one receive slot inside a window */

typedef struct fp4ar_ctx fp4ar_ctx;
typedef void* fp4ar_stream;     /* cudaStream_t */

enum { FP4AR_MODE_FUSED = 0, FP4AR_MODE_XPORT = 1, FP4AR_MODE_COMPUTE = 2 };
enum { FP4AR_ALGO_AUTO = -1, FP4AR_ALGO_ONESHOT = 0, FP4AR_ALGO_TWOSHOT = 1 };
enum { FP4AR_IN_BF16 = 0, FP4AR_IN_NVFP4 = 1, FP4AR_IN_PUSHED = 2 };
enum { FP4AR_EPI_NONE = 0, FP4AR_EPI_NORM_BF16 = 1, FP4AR_EPI_NORM_NVFP4 = 2, FP4AR_EPI_NORM_MXFP8 = 3 };

enum {
  FP4AR_OK = 0,
  FP4AR_ERR_ARGUMENT = 1,     /* bad pointer / size / enum value */
  FP4AR_ERR_UNSUPPORTED = 2,  /* combination without a kernel */
  FP4AR_ERR_CUDA = 3,         /* a CUDA runtime call failed; see fp4ar_last_cuda_error() */
  FP4AR_ERR_POISONED = 4      /* an earlier call timed out: fp4ar_reset() (collective) is required */
};

typedef struct fp4ar_args {
  const void* x;          /* IN_BF16: [rows][6144] BF16.  IN_NVFP4: [rows][3456] bytes.  IN_PUSHED: unused */
  void* out;              /* EPI_NONE / EPI_NORM_BF16: [rows][6144] BF16 */
  int rows;
  int hidden;             /* must be 6144 */
  int mode;               /* FP4AR_MODE_* */
  int algo;               /* FP4AR_ALGO_*; AUTO = one-shot up to 2 ranks, two-shot above */
  int input;              /* FP4AR_IN_* */
  int epilogue;           /* FP4AR_EPI_* */
  float gs[FP4AR_MAX_RANKS]; /* static per-rank scales of NVFP4 / pushed input, known to every rank */
  const void* res_in;     /* epilogue != NONE: [rows][6144] BF16 residual */
  void* res_out;          /* epilogue != NONE: [rows][6144] BF16, may alias res_in */
  const void* weight;     /* epilogue != NONE: [6144] BF16 */
  float eps;
  float weight_bias;      /* 1.0 for Gemma RMSNorm */
  void* outq;             /* EPI_NORM_NVFP4: [rows][3456]; EPI_NORM_MXFP8: [rows][6336] */
  float qscale;           /* EPI_NORM_NVFP4: global scale multiplied into the block scales */
  int tune[4];            /* [0] teams per CTA (0 = default), [1] bit 0: no programmatic dependent launch,
                             [2] warps per row team (0 = default: 6 for two-shot at 4 and 8 ranks, else 3; compiled widths:
                             3 for every shape, 6 for the two-shot shapes of 4 and 8 ranks),
                             [3] two-shot pipeline depths, lag_owner | lag_finish << 4 (0 = default: (2,3) with six-warp teams,
                                 (1,2) / (2,3) with three-warp teams at up to four / more ranks) */
} fp4ar_args;

typedef struct fp4ar_status_words {
  uint32_t code, row, source, detail, cta, call, count, pad;
} fp4ar_status_words;

/* Bytes of window each rank must provide for calls of up to max_rows rows.  0 = unsupported shape. */
size_t fp4ar_window_bytes(int max_rows, int hidden, int nranks);

/* windows[r] is rank r's window as addressable from this device (windows[rank] is local memory).
 * Fills the local window with sentinels and synchronises the device.  The caller must run a
 * barrier over all ranks between fp4ar_create and the first launch. */
int fp4ar_create(fp4ar_ctx** ctx, int rank, int nranks, int device, int max_rows, int hidden,
                 void* const* windows, size_t window_bytes);

/* All nranks ranks on ONE device: every launch runs the ranks as CTA groups of one cooperative
 * kernel (the groups wait on one another, so they must be co-resident).  For tests and profiling. */
int fp4ar_create_emulated(fp4ar_ctx** ctx, int nranks, int device, int max_rows, int hidden,
                          void* const* windows, size_t window_bytes);

/* args: one entry per local rank (1, or nranks for an emulated context). */
int fp4ar_launch(fp4ar_ctx* ctx, const fp4ar_args* args, fp4ar_stream stream);

/* Synchronous read of the device status block of a local rank. */
int fp4ar_status(fp4ar_ctx* ctx, int local_rank, fp4ar_status_words* out);
/* How long a device-side wait may last before it gives up (default 10000 ms, or FP4AR_TIMEOUT_MS from the
 * environment when the context is created). */
int fp4ar_set_timeout_ms(fp4ar_ctx* ctx, int ms);
/* Re-arm the whole local window and clear the status.  Collective: barrier before the next launch. */
int fp4ar_reset(fp4ar_ctx* ctx);
int fp4ar_destroy(fp4ar_ctx* ctx);

/* Geometry a producer kernel needs to push NVFP4 rows straight into the receive windows
 * (FP4AR_IN_PUSHED): slot of (source rank, row) in the window of rank `dest` for the NEXT launch. */
typedef struct fp4ar_push_view {
  uint32_t* call_counter;   /* device pointer: parity of *call_counter selects the buffer */
  size_t buffer_bytes;      /* window = 2 buffers of this size */
  int cap;                  /* rows per source in the one-shot layout */
  int capo;                 /* rows per source in the two-shot (owner) layout */
  int nranks, rank;
  void* windows[FP4AR_MAX_RANKS];
} fp4ar_push_view;
int fp4ar_get_push_view(fp4ar_ctx* ctx, int local_rank, fp4ar_push_view* out);

int fp4ar_ctas_per_rank(fp4ar_ctx* ctx);
const char* fp4ar_last_cuda_error(void);
const char* fp4ar_build_info(void);
/* Teams per CTA of the compiled kernel for this shape (0 = not compiled). */
int fp4ar_has_kernel(int nranks, int algo, int input, int epilogue, int team_warps);
/* Warps per row team a launch uses when tune[2] is 0 (algo: FP4AR_ALGO_ONESHOT / TWOSHOT, already resolved). */
int fp4ar_default_team_warps(int nranks, int algo);

/* ---- stand-alone codec / norm kernels (single GPU, no window) ---- */
int fp4ar_encode(const void* x_bf16, int rows, void* values, long values_pitch, void* scales, long scales_pitch,
                 float* row_scales, fp4ar_stream stream);
int fp4ar_encode_static(const void* x_bf16, int rows, float gs, void* qrows /* [rows][3456] */, fp4ar_stream stream);
/* sources: nsrc base pointers; values at +r*pitch, scales at +r*pitch+3072; row scales rs[s] (or NULL with gs[s]) */
int fp4ar_decode_sum(int nsrc, const void* const* src, long pitch, const float* const* rs, const float* gs, int rows,
                     void* out_bf16, fp4ar_stream stream);
/* Owner step of the two-shot algorithm as a stand-alone op: decode-sum, re-encode, decode of the re-encoding. */
int fp4ar_reduce_reencode(int nsrc, const void* const* src, long pitch, const float* const* rs, const float* gs,
                          int rows, void* rec_out /* [rows][3584] */, void* out_bf16, fp4ar_stream stream);
int fp4ar_add_rmsnorm(const void* x_bf16, const void* res_in, void* res_out, const void* weight, float eps,
                      float weight_bias, int epilogue, float qscale, void* out_bf16, void* outq, int rows,
                      fp4ar_stream stream);
/* window = nbuffers buffers of buffer_bytes each; receive slots start at every buffer's first byte */
int fp4ar_fill_sentinel(void* window, size_t buffer_bytes, int nbuffers, fp4ar_stream stream);

/* Exhaustive check of the encoder's division-free multiplier for one exponent of the row-scale inverse (27..227):
 * adds the number of (mantissa, scale byte) cases that differ from IEEE division to *device_mismatch_counter. */
int fp4ar_selftest_scale_division(int exp_biased, unsigned long long* device_mismatch_counter, fp4ar_stream stream);
/* Exhaustive checks of the hardware conversions against plain software models; mismatches are added to the counter.
 * which 0: E4M3 block scale of x / 6 for the non-negative FP32 bit patterns [first, first + count) (domain 0 .. 2^31);
 * which 1: E2M1 value encode for the FP32 bit patterns [first, first + count) in every nibble position;
 * which 2: E2M1 / E4M3 decode tables and the -0 canonicalisation (first, count ignored).  count 0 = to the end.
 * which 3 / 4: `count` pseudo-random BF16 / FP32 pairs (seed `first`): the table-driven block encoder against the one
 *          with IEEE divisions; counter[0] += mismatching words, counter[1] += sentinels produced (two counters);
 * which 5: `count` (<= 2^17) rounds of 2^14 decode-accumulate cases, one per pair of non-negative scale bytes,
 *          against scalar table arithmetic. */
int fp4ar_selftest_conversions(int which, unsigned int first, unsigned int count,
                               unsigned long long* device_mismatch_counter, fp4ar_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* FP4AR_H_ */
