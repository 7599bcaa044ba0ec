/*
 * pi05_b200 — C ABI of the B200-native PI0.5 policy-forward library.
 *
 * Plain C: device/host pointers, integer sizes, integer status returns. Every
 * entry point returns 0 on success and a negative Pi05Status on failure; no
 * entry point throws, aborts or falls back to a CPU path. Launch functions do
 * not allocate device memory unless their comment says so.
 *
 * Two levels, mirroring the reference (infinigence/ApxInf):
 *   - engine level: what `pi05_bench` and the `apxinf-model` PI0.5 runtime
 *     expose (crates/apxinf-model/src/pi05/{bf16_runtime,runtime,int8_runtime}.rs);
 *   - kernel level: what `crates/apxinf-cuda/src/ffi/*.rs` binds.
 */
#ifndef PI05_B200_H_
#define PI05_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum Pi05Status {
  PI05_OK = 0,
  PI05_ERR_INVALID_VALUE = -1,  /* bad argument, rejected before any launch */
  PI05_ERR_UNSUPPORTED = -2,    /* legal but not built (shape / dtype combination) */
  PI05_ERR_DRIVER = -3,         /* CUDA driver entry point missing or tensor-map encode failed */
  PI05_ERR_CUDA = -4,           /* a CUDA runtime call failed; see pi05_last_cuda_error() */
  PI05_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait ran out (status word != 0) */
  PI05_ERR_NOT_BUILT = -6
} Pi05Status;

/* Operand / output element types and fused epilogues of pi05_gemm. */
enum { PI05_OP_BF16 = 0, PI05_OP_E4M3 = 1, PI05_OP_S8 = 2 };
enum { PI05_OUT_BF16 = 0, PI05_OUT_E4M3 = 1, PI05_OUT_F32 = 2, PI05_OUT_S32 = 3 };
enum {
  PI05_EPI_STORE = 0,
  PI05_EPI_BIAS_GELU = 1,
  PI05_EPI_BIAS_SILU = 2,
  PI05_EPI_BIAS_RESIDUAL = 3,
  PI05_EPI_BIAS_POS = 4,
  PI05_EPI_GATE_RESIDUAL = 5,
  PI05_EPI_GEGLU = 6
};

/*
 * One dense linear layer out[M, N] = epilogue(a[M, K] . b[N, K]^T) on the
 * tcgen05 tensor cores. `a` and `b` are K-major device matrices (leading
 * dimensions in elements, rows 16-byte aligned); with b_mn_major != 0, `b` is a
 * row-major [K, N] matrix instead. Batched over nb0 x nb1 with element strides.
 * Replaces the reference GEMM contracts gemm::bf16 / gemm::fp8 / gemm::w8a8 and
 * their fused variants (crates/apxinf-cuda/src/kernels/gemm/bf16.rs:355-453,
 * fp8.rs:457-617, w8a8.rs:30-152, crates/apxinf-cuda/src/kernels/fused.rs:18-119)
 * and the FFI symbols behind them (crates/apxinf-cuda/src/ffi/cublaslt.rs:55,112,
 * ffi/cutlass.rs:85-160).
 */
typedef struct Pi05GemmArgs {
  int32_t op;          /* PI05_OP_* of both operands */
  int32_t m, n, k;
  int32_t nb0, nb1;    /* batch extents (>= 1) */
  const void* a;
  int64_t lda, a_sb0, a_sb1;
  const void* b;
  int64_t ldb, b_sb0, b_sb1;
  int32_t b_mn_major;
  void* out;
  int64_t ldc, out_sb0, out_sb1;
  int32_t out_type;    /* PI05_OUT_* */
  int32_t mode;        /* PI05_EPI_* */
  const void* residual;   /* bf16, same geometry as out */
  const void* bias;       /* bf16 [n] */
  const float* col_scale; /* f32 [n], per-output-channel weight scale, or NULL */
  const float* row_scale; /* f32 [m], per-row activation scale, or NULL */
  const void* pos;        /* bf16 [pos_rows, n] */
  int32_t pos_rows;
  int64_t pos_ld;
  const void* gate;       /* bf16 [n] */
  float alpha;
  float out_inv_scale;
  int32_t* status;        /* device int32, must be 0 before the call; set on device timeouts */
  int32_t force_swap;     /* -1 auto */
  int32_t force_block_n;  /* 0 auto */
} Pi05GemmArgs;

int pi05_gemm(const Pi05GemmArgs* args, void* cuda_stream);

/* Last CUDA runtime error string seen by this library on the calling thread. */
const char* pi05_last_cuda_error(void);

/* Library build identification: "pi05_b200 sm_100a <date>". */
const char* pi05_version(void);

#ifdef __cplusplus
}
#endif

#endif /* PI05_B200_H_ */
