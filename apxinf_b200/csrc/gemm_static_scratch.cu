// pi05_gemm_static_scratch: the split-K GEMM for callers that cannot allocate.
//
// The scratch a split-K launch needs (one raw accumulator tile per split and output
// tile, plus an arrival counter per output tile) is a fixed array in this library's
// image, so the call never touches an allocator. The array's name is only a
// host-side stand-in: the kernel gets the address cudaGetSymbolAddress reports for
// the device that is current, looked up once per device in this file.
#include <mutex>
#include <string>

#include "../../include/pi05_b200.h"
#include "gemm.h"

namespace pi05 {
extern thread_local std::string g_last_cuda_error;
int record_cuda(cudaError_t error);
}  // namespace pi05

namespace {

constexpr int kMaxDevices = 64;

struct StaticScratch {
  unsigned char partials[PI05_STATIC_SCRATCH_BYTES];
  int counters[PI05_STATIC_SCRATCH_TILES];
};

// One copy per GPU that loads the library, zero-initialised at module load.
static __device__ __align__(256) StaticScratch g_static_scratch;

std::mutex g_lookup_mutex;
StaticScratch* g_device_address[kMaxDevices] = {};

// Device address of the scratch on the current device; first use per device asks the
// runtime (not capturable: do it before any stream capture).
int scratch_for_current_device(StaticScratch** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return pi05::record_cuda(err);
  if (device < 0 || device >= kMaxDevices) return pi05::kPi05ErrInvalidValue;
  std::lock_guard<std::mutex> lock(g_lookup_mutex);
  if (g_device_address[device] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_scratch);
    if (err != cudaSuccess) return pi05::record_cuda(err);
    if (address == nullptr) return pi05::kPi05ErrCuda;
    g_device_address[device] = static_cast<StaticScratch*>(address);
  }
  *out = g_device_address[device];
  return pi05::kPi05Ok;
}

}  // namespace

extern "C" int pi05_gemm_static_scratch(const Pi05GemmArgs* args, void* cuda_stream) {
  using namespace pi05;
  if (args == nullptr) return kPi05ErrInvalidValue;
  if (args->force_split_k < 2) {
    g_last_cuda_error = "pi05_gemm_static_scratch is the split-K variant: force_split_k must be >= 2";
    return kPi05ErrInvalidValue;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The scratch address is the current device's copy: a stream of another device would run
  // the kernel there with this device's pointer.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread &&
      cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) {
    return record_cuda(cudaGetLastError());
  }
  // (a capturing stream is not asked for its device: the query is not a capturable call)
  if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread &&
      capturing == cudaStreamCaptureStatusNone) {
    int current = -1, stream_device = -1;
    cudaError_t err = cudaGetDevice(&current);
    if (err == cudaSuccess) err = cudaStreamGetDevice(stream, &stream_device);
    if (err != cudaSuccess) return record_cuda(err);
    if (current != stream_device) {
      g_last_cuda_error = "pi05_gemm_static_scratch: the stream belongs to device " +
                          std::to_string(stream_device) + " but device " + std::to_string(current) +
                          " is current";
      return kPi05ErrInvalidValue;
    }
  }
  StaticScratch* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != kPi05Ok) return rc;

  GemmProblem q;
  q.op = args->op;
  q.M = args->m;
  q.N = args->n;
  q.K = args->k;
  q.nb0 = args->nb0;
  q.nb1 = args->nb1;
  q.a = GemmOperand{args->a, args->m, args->lda, args->a_sb0, args->a_sb1};
  q.b = GemmOperand{args->b, args->b_mn_major ? args->k : args->n, args->ldb, args->b_sb0,
                    args->b_sb1};
  q.b_mn_major = args->b_mn_major != 0;
  q.out = args->out;
  q.ldc = args->ldc;
  q.out_sb0 = args->out_sb0;
  q.out_sb1 = args->out_sb1;
  q.out_type = args->out_type;
  q.mode = args->mode;
  q.residual = args->residual;
  q.bias = args->bias;
  q.col_scale = args->col_scale;
  q.row_scale = args->row_scale;
  q.pos = args->pos;
  q.pos_rows = args->pos_rows;
  q.pos_ld = args->pos_ld;
  q.gate = args->gate;
  q.alpha = args->alpha;
  q.out_inv_scale = args->out_inv_scale;
  q.status = args->status;
  q.force_swap = args->force_swap;
  q.force_block_n = args->force_block_n;
  q.force_split_k = args->force_split_k;
  q.b_blocked = args->b_blocked != 0;
  q.force_skinny = 0;  // this entry point is the split-K tcgen05 variant
  q.partials = scratch->partials;
  q.partials_bytes = PI05_STATIC_SCRATCH_BYTES;
  q.tile_counters = scratch->counters;
  q.max_tiles = PI05_STATIC_SCRATCH_TILES;

  GemmPlan plan;
  rc = gemm_plan_build(q, &plan);
  if (rc == kPi05ErrScratchLimit) {
    g_last_cuda_error = "split-K request exceeds the built-in scratch (" +
                        std::to_string(PI05_STATIC_SCRATCH_BYTES) + " bytes of partial tiles, " +
                        std::to_string(PI05_STATIC_SCRATCH_TILES) +
                        " output tiles): use fewer splits or pi05_gemm with caller scratch";
    return rc;
  }
  if (rc != kPi05Ok) return rc;
  // The array keeps whatever the last call left; the arrival counters must start at zero.
  cudaError_t err = cudaMemsetAsync(scratch->counters, 0, sizeof(scratch->counters), stream);
  if (err != cudaSuccess) return record_cuda(err);
  return record_cuda(gemm_plan_launch(plan, stream));
}
