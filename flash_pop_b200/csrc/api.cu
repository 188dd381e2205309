// extern "C" entry points of flash_pop_b200: argument validation, choice between the tcgen05
// kernels and the CUDA-core kernels, launches.  Declarations and the reference interfaces each
// entry point replaces are in include/flash_pop_b200.h.
#include <atomic>
#include <cmath>
#include <cstring>

#include "fpb_common.cuh"
#include "umma_launch.h"

namespace fpb {

__device__ int32_t g_device_status = 0;

int32_t* device_status_ptr() {
  // one address per device; a handful of devices at most
  static std::atomic<int32_t*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int32_t* p = cache[dev].load(std::memory_order_acquire);
  if (!p) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_device_status) != cudaSuccess) return nullptr;
    p = (int32_t*)sym;
    cache[dev].store(p, std::memory_order_release);
  }
  return p;
}

// Scratch memory that belongs to the library image itself, for fpb_retention_fwd_static: callers that must not allocate
// get the T-segment scratch from here.  Every device that loads the library holds these bytes until the process exits.
// In host code the array's name is only a stand-in for the symbol - not a device address, a kernel must never be given
// it - so the address is asked for once per device (static_scratch_ptr) and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_static_scratch[FPB_STATIC_SCRATCH_BYTES];

namespace {

// Device address of g_static_scratch on the current device: looked up on the first call per device, with that device
// current, and kept.  Null if the runtime refuses.
float* static_scratch_ptr() {
  static std::atomic<float*> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  float* p = cache[dev].load(std::memory_order_acquire);
  if (!p) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_static_scratch) != cudaSuccess || !sym) { cudaGetLastError(); return nullptr; }
    p = (float*)sym;
    cache[dev].store(p, std::memory_order_release);
  }
  return p;
}

thread_local int tl_last_path = FPB_PATH_NONE;
thread_local int tl_last_cuda_error = 0;
std::atomic<int64_t> g_launches{0};

struct Call {
  int dtype, B, T, H, dk, dv, block_size, n_blocks, flags;
  bool state_f32;            // states are fp32 (always so for fp32 activations)
  float* scratch; int64_t scratch_bytes;
  float gamma[FPB_MAX_HEADS];
  bool tensor_core_decays;   // every decay large enough for the gamma^-L rescaling of the tcgen05 path
};

SeqView view(const fpb_seq* s) { return s ? SeqView{s->data, s->stride_b, s->stride_t, s->stride_h} : SeqView{nullptr, 0, 0, 0}; }
StateView view(const fpb_state* s) { return s ? StateView{s->data, s->stride_b, s->stride_h} : StateView{nullptr, 0, 0}; }

int check_device() {
  static std::atomic<int> ok[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FPB_ERR_NO_DEVICE_CODE;
  // Tensor maps are encoded through the driver API, which needs the device's primary context current
  // on the calling host thread; a thread that has made no runtime call yet (an autograd worker, say)
  // has none.  cudaSetDevice binds it.
  thread_local int bound = -1;
  if (bound != dev) {
    if (cudaSetDevice(dev) != cudaSuccess) return FPB_ERR_NO_DEVICE_CODE;
    bound = dev;
  }
  if (dev >= 0 && dev < 64 && ok[dev].load()) return FPB_OK;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10)
    return FPB_ERR_NO_DEVICE_CODE;
  if (dev >= 0 && dev < 64) ok[dev].store(1);
  return FPB_OK;
}

int check_dims(const fpb_dims* d, bool pop, Call* c) {
  if (!d) return FPB_ERR_NULL_POINTER;
  if (d->dtype != FPB_BF16 && d->dtype != FPB_F32) return FPB_ERR_BAD_DTYPE;
  if (d->B < 0 || d->T < 0 || d->H < 0 || d->dk <= 0 || d->dv <= 0) return FPB_ERR_BAD_SHAPE;
  if (d->H > FPB_MAX_HEADS || d->dk > 256 || d->dv > 256) return FPB_ERR_BAD_SHAPE;
  if (pop && d->block_size <= 0) return FPB_ERR_BAD_BLOCK_SIZE;
  if (d->H > 0 && !d->head_decays) return FPB_ERR_NULL_POINTER;
  c->dtype = d->dtype; c->B = d->B; c->T = d->T; c->H = d->H; c->dk = d->dk; c->dv = d->dv;
  c->flags = d->flags;
  c->state_f32 = d->dtype == FPB_F32 || (d->flags & FPB_FLAG_STATE_F32) != 0;
  if (d->workspace_bytes < 0 || (uintptr_t)d->workspace % 16) return FPB_ERR_BAD_WORKSPACE;
  c->scratch = (d->workspace && d->workspace_bytes > 0) ? (float*)d->workspace : nullptr;
  c->scratch_bytes = c->scratch ? d->workspace_bytes : 0;
  c->block_size = pop ? d->block_size : 0;
  c->n_blocks = pop ? d->T / d->block_size : 0;
  c->tensor_core_decays = true;
  for (int h = 0; h < d->H; ++h) {
    const double g = d->head_decays[h];
    if (!std::isfinite(g) || g < 0.0 || g > 1.0) return FPB_ERR_BAD_DECAY;
    c->gamma[h] = (float)g;              // the reference rounds gamma to fp32 before any power
    if (g < 0.5) c->tensor_core_decays = false;
  }
  return FPB_OK;
}

int check_seq(const Call& c, const fpb_seq* s, int d, int64_t batch, bool optional = false) {
  if (optional && (!s || !s->data)) return FPB_OK;
  if (!s) return FPB_ERR_NULL_POINTER;
  const bool empty = batch == 0 || c.T == 0 || c.H == 0;
  if (!s->data) return empty ? FPB_OK : FPB_ERR_NULL_POINTER;
  if ((batch > 1 && s->stride_b <= 0) || (c.T > 1 && s->stride_t <= 0) || (c.H > 1 && s->stride_h < d))
    return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}

int check_state(const fpb_state* s, const Call& c) {
  if (!s || !s->data) return FPB_OK;
  const int64_t blk = (int64_t)c.dk * c.dv;
  if ((c.H > 1 && s->stride_h < blk) || (c.B > 1 && s->stride_b < blk)) return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}

int finish_launches(int n, int path) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { tl_last_cuda_error = (int)e; return FPB_ERR_LAUNCH; }
  g_launches.fetch_add(n);
  if (path >= 0) tl_last_path = path;   // the elementwise entry points pass -1 and leave the operator's record alone
  return FPB_OK;
}

void fill_common(WalkParams& p, const Call& c, int dir, const SuffixStates& sfx) {
  std::memset(&p, 0, sizeof(p));
  p.T = c.T; p.H = c.H; p.dk = c.dk; p.dv = c.dv; p.dir = dir;
  p.block_size = c.block_size; p.n_blocks = c.n_blocks;
  p.scale_u = p.scale_w = p.scale_r = p.scale_out = 1.0f;
  p.sfx = sfx;
  std::memcpy(p.gamma, c.gamma, sizeof(float) * c.H);
}

void own_is_dv(WalkParams& p, const Call& c) { p.n_own = c.dv; p.n_red = c.dk; p.x_stride_red = c.dv; p.x_stride_own = 1; }
void own_is_dk(WalkParams& p, const Call& c) { p.n_own = c.dk; p.n_red = c.dv; p.x_stride_red = 1; p.x_stride_own = c.dv; }

// ---- forward (plain, POP, suffix) --------------------------------------------------------------
int forward(const Call& c, int64_t batch, SeqView q, SeqView k, SeqView v, StateView s0, SeqView o, StateView s_out,
            void* block_states, SuffixStates sfx, cudaStream_t stream) {
  if (batch == 0 || c.H == 0) return FPB_OK;
  const float rs = 1.0f / sqrtf((float)c.dk);
  if (!(c.flags & FPB_FLAG_FORCE_SIMT) && c.tensor_core_decays && c.T > 0) {
    UmmaFwdArgs a{};
    a.q = q; a.k = k; a.v = v; a.o = o; a.s0 = s0; a.s_out = s_out; a.block_states = block_states; a.sfx = sfx;
    a.B = (int)batch; a.T = c.T; a.H = c.H; a.dk = c.dk; a.dv = c.dv; a.dtype = c.dtype;
    a.block_size = c.block_size; a.n_blocks = c.n_blocks; a.gamma = c.gamma;
    a.state_f32 = c.state_f32; a.scratch = c.scratch; a.scratch_bytes = c.scratch_bytes;
    int n_launched = 0;
    const int r = launch_umma_fwd(a, stream, &n_launched);
    if (r == FPB_OK) return finish_launches(n_launched, FPB_PATH_TCGEN05);
    if (r != FPB_UMMA_NOT_APPLICABLE) return r;
  }
  WalkParams p;
  fill_common(p, c, +1, sfx);
  own_is_dv(p, c);
  p.u = v; p.w = k; p.r = q; p.out = o; p.scale_w = rs;
  p.x0 = s0; p.x_out = s_out; p.block_out = block_states;
  const int r = launch_walk(p, c.dtype, c.state_f32, (int)batch, stream);
  return r != FPB_OK ? r : finish_launches(1, FPB_PATH_SIMT);
}

// ---- backward (plain, POP, suffix) -------------------------------------------------------------
int backward(const Call& c, int64_t batch, SeqView q, SeqView k, SeqView v, StateView s0, SeqView dO, StateView d_s_out,
             const void* d_block_states, SeqView dQ, SeqView dK, SeqView dV, StateView d_s0, SuffixStates sfx_in,
             SuffixStates sfx_grad, cudaStream_t stream) {
  if (batch == 0 || c.H == 0) return FPB_OK;
  const float rs = 1.0f / sqrtf((float)c.dk);
  if (!(c.flags & FPB_FLAG_FORCE_SIMT) && c.tensor_core_decays && c.T > 0) {
    UmmaBwdArgs a{};
    a.q = q; a.k = k; a.v = v; a.dO = dO; a.dQ = dQ; a.dK = dK; a.dV = dV;
    a.s0 = s0; a.d_s_out = d_s_out; a.d_s0 = d_s0; a.d_block_states = d_block_states;
    a.sfx_in = sfx_in; a.sfx_grad = sfx_grad;
    a.B = (int)batch; a.T = c.T; a.H = c.H; a.dk = c.dk; a.dv = c.dv; a.dtype = c.dtype;
    a.block_size = c.block_size; a.n_blocks = c.n_blocks; a.gamma = c.gamma;
    a.skip_dq = (c.flags & FPB_FLAG_SKIP_DQ) != 0; a.skip_dkdv = (c.flags & FPB_FLAG_SKIP_DKDV) != 0;
    a.state_f32 = c.state_f32; a.scratch = c.scratch; a.scratch_bytes = c.scratch_bytes;
    int n_launched = 0;
    const int r = launch_umma_bwd(a, stream, &n_launched);
    if (r == FPB_OK) return finish_launches(n_launched, FPB_PATH_TCGEN05);
    if (r != FPB_UMMA_NOT_APPLICABLE) return r;
  }
  WalkParams p;
  int r, n = 0;
  if (!(c.flags & FPB_FLAG_SKIP_DQ)) {
    // dQ: forward walk over the states
    fill_common(p, c, +1, sfx_in);
    own_is_dk(p, c);
    p.u = k; p.w = v; p.r = dO; p.out = dQ; p.scale_u = rs; p.x0 = s0;
    if ((r = launch_walk(p, c.dtype, c.state_f32, (int)batch, stream)) != FPB_OK) return r;
    ++n;
  }
  if (!(c.flags & FPB_FLAG_SKIP_DKDV)) {
    // dV and dS_0: reverse walk over the state gradient
    fill_common(p, c, -1, sfx_grad);
    own_is_dv(p, c);
    p.u = dO; p.w = q; p.r = k; p.out = dV; p.scale_r = rs;
    p.x0 = d_s_out; p.x_out = d_s0; p.block_in = d_block_states;
    if ((r = launch_walk(p, c.dtype, c.state_f32, (int)batch, stream)) != FPB_OK) return r;
    // dK: reverse walk, transposed ownership
    SuffixStates no_write = sfx_grad;
    no_write.blocks = nullptr;
    fill_common(p, c, -1, no_write);
    own_is_dk(p, c);
    p.u = q; p.w = dO; p.r = v; p.out = dK; p.scale_out = rs;
    p.x0 = d_s_out; p.block_in = d_block_states;
    if ((r = launch_walk(p, c.dtype, c.state_f32, (int)batch, stream)) != FPB_OK) return r;
    n += 2;
  }
  return finish_launches(n, FPB_PATH_SIMT);
}

}  // namespace
}  // namespace fpb

using namespace fpb;

#define FPB_TRY(expr) do { const int _s = (expr); if (_s != FPB_OK) return _s; } while (0)

extern "C" {

int fpb_retention_fwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                      const fpb_state* s0, const fpb_seq* o, const fpb_state* s_out, fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B));
  FPB_TRY(check_seq(c, v, c.dv, c.B)); FPB_TRY(check_seq(c, o, c.dv, c.B));
  FPB_TRY(check_state(s0, c)); FPB_TRY(check_state(s_out, c));
  FPB_TRY(check_device());
  return forward(c, c.B, view(q), view(k), view(v), view(s0), view(o), view(s_out), nullptr, SuffixStates{0, 0, nullptr},
                 (cudaStream_t)stream);
}

int fpb_retention_fwd_static(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                             const fpb_state* s0, const fpb_seq* o, const fpb_state* s_out, fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  if (dims->workspace) return FPB_ERR_BAD_WORKSPACE;      // this entry point brings its own scratch
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B));
  FPB_TRY(check_seq(c, v, c.dv, c.B)); FPB_TRY(check_seq(c, o, c.dv, c.B));
  FPB_TRY(check_state(s0, c)); FPB_TRY(check_state(s_out, c));
  FPB_TRY(check_device());
  // a shape whose full split needs more than the built-in scratch holds is refused rather than split less
  if (fpb_workspace_bytes(dims) > (int64_t)FPB_STATIC_SCRATCH_BYTES) return FPB_ERR_TOO_LARGE;
  float* scratch = static_scratch_ptr();
  if (!scratch) { tl_last_cuda_error = (int)cudaErrorInvalidSymbol; return FPB_ERR_LAUNCH; }
  c.scratch = scratch;
  c.scratch_bytes = FPB_STATIC_SCRATCH_BYTES;
  return forward(c, c.B, view(q), view(k), view(v), view(s0), view(o), view(s_out), nullptr, SuffixStates{0, 0, nullptr},
                 (cudaStream_t)stream);
}

int fpb_copy_rows_async(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes, int64_t rows,
                        fpb_stream_t stream) {
  if (rows == 0 || width_bytes == 0) return FPB_OK;
  if (!dst || !src) return FPB_ERR_NULL_POINTER;
  if (rows < 0 || width_bytes < 0 || dst_pitch < width_bytes || src_pitch < width_bytes) return FPB_ERR_BAD_STRIDE;
  if (cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes, (size_t)rows, cudaMemcpyDefault,
                        (cudaStream_t)stream) != cudaSuccess) {
    tl_last_cuda_error = (int)cudaGetLastError();
    return FPB_ERR_LAUNCH;
  }
  return FPB_OK;
}

int fpb_retention_bwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                      const fpb_state* s0, const fpb_seq* d_o, const fpb_state* d_s_out,
                      const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                      fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B)); FPB_TRY(check_seq(c, v, c.dv, c.B));
  FPB_TRY(check_seq(c, d_o, c.dv, c.B));
  FPB_TRY(check_seq(c, d_q, c.dk, c.B, c.flags & FPB_FLAG_SKIP_DQ));
  FPB_TRY(check_seq(c, d_k, c.dk, c.B, c.flags & FPB_FLAG_SKIP_DKDV)); FPB_TRY(check_seq(c, d_v, c.dv, c.B, c.flags & FPB_FLAG_SKIP_DKDV));
  FPB_TRY(check_state(s0, c)); FPB_TRY(check_state(d_s_out, c)); FPB_TRY(check_state(d_s0, c));
  FPB_TRY(check_device());
  const SuffixStates none{0, 0, nullptr};
  return backward(c, c.B, view(q), view(k), view(v), view(s0), view(d_o), view(d_s_out), nullptr, view(d_q), view(d_k),
                  view(d_v), view(d_s0), none, none, (cudaStream_t)stream);
}

int fpb_pop_retention_fwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                          const fpb_state* s0, const fpb_seq* o, void* block_states, fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, true, &c));
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B));
  FPB_TRY(check_seq(c, v, c.dv, c.B)); FPB_TRY(check_seq(c, o, c.dv, c.B));
  FPB_TRY(check_state(s0, c));
  if (c.n_blocks > 0 && c.B > 0 && c.H > 0 && !block_states) return FPB_ERR_NULL_POINTER;
  FPB_TRY(check_device());
  return forward(c, c.B, view(q), view(k), view(v), view(s0), view(o), StateView{nullptr, 0, 0}, block_states,
                 SuffixStates{0, 0, nullptr}, (cudaStream_t)stream);
}

int fpb_pop_retention_bwd(const fpb_dims* dims, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                          const fpb_state* s0, const fpb_seq* d_o, const void* d_block_states,
                          const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                          fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, true, &c));
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B)); FPB_TRY(check_seq(c, v, c.dv, c.B));
  FPB_TRY(check_seq(c, d_o, c.dv, c.B));
  FPB_TRY(check_seq(c, d_q, c.dk, c.B, c.flags & FPB_FLAG_SKIP_DQ));
  FPB_TRY(check_seq(c, d_k, c.dk, c.B, c.flags & FPB_FLAG_SKIP_DKDV)); FPB_TRY(check_seq(c, d_v, c.dv, c.B, c.flags & FPB_FLAG_SKIP_DKDV));
  FPB_TRY(check_state(s0, c)); FPB_TRY(check_state(d_s0, c));
  FPB_TRY(check_device());
  const SuffixStates none{0, 0, nullptr};
  return backward(c, c.B, view(q), view(k), view(v), view(s0), view(d_o), StateView{nullptr, 0, 0}, d_block_states,
                  view(d_q), view(d_k), view(d_v), view(d_s0), none, none, (cudaStream_t)stream);
}

int fpb_pop_suffix_fwd(const fpb_dims* dims, int32_t M, int32_t N, const fpb_seq* q, const fpb_seq* k,
                       const fpb_seq* v, const fpb_state* s0, const void* block_states, const fpb_seq* o,
                       fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  if (M < 0 || N < 0 || M > N + 1) return FPB_ERR_BAD_SHAPE;
  const int64_t batch = (int64_t)c.B * M;
  if (batch > 0x7fffffff) return FPB_ERR_TOO_LARGE;
  FPB_TRY(check_seq(c, q, c.dk, batch)); FPB_TRY(check_seq(c, k, c.dk, batch));
  FPB_TRY(check_seq(c, v, c.dv, batch)); FPB_TRY(check_seq(c, o, c.dv, batch));
  FPB_TRY(check_state(s0, c));
  if (M > 1 && c.B > 0 && c.H > 0 && !block_states) return FPB_ERR_NULL_POINTER;
  FPB_TRY(check_device());
  if (M == 0) return FPB_OK;
  return forward(c, batch, view(q), view(k), view(v), view(s0), view(o), StateView{nullptr, 0, 0}, nullptr,
                 SuffixStates{M, N, const_cast<void*>(block_states)}, (cudaStream_t)stream);
}

int fpb_pop_suffix_bwd(const fpb_dims* dims, int32_t M, int32_t N, const fpb_seq* q, const fpb_seq* k,
                       const fpb_seq* v, const fpb_state* s0, const void* block_states, const fpb_seq* d_o,
                       const fpb_seq* d_q, const fpb_seq* d_k, const fpb_seq* d_v, const fpb_state* d_s0,
                       void* d_block_states, fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  if (M < 0 || N < 0 || M > N + 1) return FPB_ERR_BAD_SHAPE;
  const int64_t batch = (int64_t)c.B * M;
  if (batch > 0x7fffffff) return FPB_ERR_TOO_LARGE;
  FPB_TRY(check_seq(c, q, c.dk, batch)); FPB_TRY(check_seq(c, k, c.dk, batch)); FPB_TRY(check_seq(c, v, c.dv, batch));
  FPB_TRY(check_seq(c, d_o, c.dv, batch));
  FPB_TRY(check_seq(c, d_q, c.dk, batch, c.flags & FPB_FLAG_SKIP_DQ));
  FPB_TRY(check_seq(c, d_k, c.dk, batch, c.flags & FPB_FLAG_SKIP_DKDV)); FPB_TRY(check_seq(c, d_v, c.dv, batch, c.flags & FPB_FLAG_SKIP_DKDV));
  FPB_TRY(check_state(s0, c)); FPB_TRY(check_state(d_s0, c));
  if (M > 1 && c.B > 0 && c.H > 0 && (!block_states || !d_block_states)) return FPB_ERR_NULL_POINTER;
  FPB_TRY(check_device());
  if (c.B == 0 || c.H == 0) return FPB_OK;
  const size_t esize = c.state_f32 ? 4 : 2;
  const size_t blk = (size_t)c.H * c.dk * c.dv * esize;
  // blocks that no suffix starts from get a zero gradient
  if (d_block_states && N > 0) {
    const int used = M > 0 ? M - 1 : 0;
    if (used < N) {
      if (cudaMemset2DAsync((char*)d_block_states + used * blk, (size_t)N * blk, 0, (size_t)(N - used) * blk, c.B,
                            (cudaStream_t)stream) != cudaSuccess)
        return finish_launches(0, FPB_PATH_NONE);
    }
  }
  if (M == 0) {
    if (d_s0 && d_s0->data) {
      for (int b = 0; b < c.B; ++b)
        cudaMemset2DAsync((char*)d_s0->data + b * d_s0->stride_b * esize, d_s0->stride_h * esize, 0,
                          (size_t)c.dk * c.dv * esize, c.H, (cudaStream_t)stream);
    }
    return finish_launches(0, FPB_PATH_NONE);
  }
  return backward(c, batch, view(q), view(k), view(v), view(s0), view(d_o), StateView{nullptr, 0, 0}, nullptr, view(d_q),
                  view(d_k), view(d_v), view(d_s0), SuffixStates{M, N, const_cast<void*>(block_states)},
                  SuffixStates{M, N, d_block_states}, (cudaStream_t)stream);
}

int fpb_retention_step(const fpb_dims* dims, int32_t state_dtype, const fpb_seq* q, const fpb_seq* k, const fpb_seq* v,
                       const fpb_state* s_prev, const fpb_seq* o, const fpb_state* s_out, fpb_stream_t stream) {
  Call c;
  FPB_TRY(check_dims(dims, false, &c));
  if (c.T != 1) return FPB_ERR_BAD_SHAPE;
  if (state_dtype != FPB_BF16 && state_dtype != FPB_F32) return FPB_ERR_BAD_DTYPE;
  if ((int64_t)c.B * c.H > 0x7fffffff) return FPB_ERR_TOO_LARGE;
  FPB_TRY(check_seq(c, q, c.dk, c.B)); FPB_TRY(check_seq(c, k, c.dk, c.B));
  FPB_TRY(check_seq(c, v, c.dv, c.B)); FPB_TRY(check_seq(c, o, c.dv, c.B));
  FPB_TRY(check_state(s_prev, c)); FPB_TRY(check_state(s_out, c));
  FPB_TRY(check_device());
  if (c.B == 0 || c.H == 0) return FPB_OK;
  launch_retention_step(c.dtype, state_dtype, c.B, c.H, c.dk, c.dv, c.gamma, view(q), view(k), view(v), view(o),
                        view(s_prev), view(s_out), (cudaStream_t)stream);
  return finish_launches(1, FPB_PATH_SIMT);
}

namespace {
// shapes and alignment of a (B,T,H,d) tensor read or written `vec` elements at a time
int check_plain_seq(const fpb_seq* s, int dtype, int B, int T, int H, int d, int vec_bytes) {
  if (!s) return FPB_ERR_NULL_POINTER;
  if (B == 0 || T == 0 || H == 0) return FPB_OK;
  if (!s->data) return FPB_ERR_NULL_POINTER;
  const int64_t vec = vec_bytes / (dtype == FPB_F32 ? 4 : 2);
  if ((B > 1 && s->stride_b <= 0) || (T > 1 && s->stride_t <= 0) || (H > 1 && s->stride_h < d)) return FPB_ERR_BAD_STRIDE;
  if ((uintptr_t)s->data % vec_bytes || s->stride_b % vec || s->stride_t % vec || s->stride_h % vec) return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}
bool dtype_ok(int t) { return t == FPB_BF16 || t == FPB_F32; }
}  // namespace

int fpb_rotary(int32_t B, int32_t T, int32_t H, int32_t d, int32_t in_dtype, int32_t out_dtype, int32_t conjugate,
               const float* phasors, int64_t phasor_stride_b, const fpb_seq* q_in, const fpb_seq* k_in,
               const fpb_seq* q_out, const fpb_seq* k_out, fpb_stream_t stream) {
  if (B < 0 || T < 0 || H < 0 || d <= 0 || d % 8) return FPB_ERR_BAD_SHAPE;
  if ((int64_t)B * T * H * (d / 8) >= (1ll << 31)) return FPB_ERR_TOO_LARGE;
  if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype)) return FPB_ERR_BAD_DTYPE;
  if ((int64_t)B * T * H * d > 0 && !phasors) return FPB_ERR_NULL_POINTER;
  if ((uintptr_t)phasors % 16 || phasor_stride_b % 2 || phasor_stride_b < 0) return FPB_ERR_BAD_STRIDE;
  FPB_TRY(check_plain_seq(q_in, in_dtype, B, T, H, d, 16)); FPB_TRY(check_plain_seq(q_out, out_dtype, B, T, H, d, 16));
  const bool two = k_in && k_in->data;
  if (two) { FPB_TRY(check_plain_seq(k_in, in_dtype, B, T, H, d, 16)); FPB_TRY(check_plain_seq(k_out, out_dtype, B, T, H, d, 16)); }
  FPB_TRY(check_device());
  if ((int64_t)B * T * H == 0) return FPB_OK;
  const SeqView in[2] = {view(q_in), two ? view(k_in) : view(q_in)}, out[2] = {view(q_out), two ? view(k_out) : view(q_out)};
  launch_rotary(in_dtype, out_dtype, B, T, H, d, conjugate != 0, phasors, phasor_stride_b, in, out, two ? 2 : 1, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_groupnorm_gate_fwd(int32_t B, int32_t T, int32_t H, int32_t dv, int32_t dtype, float eps, int32_t swish,
                           const fpb_seq* o, const fpb_seq* z, const fpb_seq* y, fpb_stream_t stream) {
  if (B < 0 || T < 0 || H < 0 || dv <= 0 || dv % 2 || dv > 256) return FPB_ERR_BAD_SHAPE;
  if ((int64_t)B * T * H >= (1ll << 31)) return FPB_ERR_TOO_LARGE;
  if (!dtype_ok(dtype)) return FPB_ERR_BAD_DTYPE;
  const int vb = dtype == FPB_F32 ? 8 : 4;
  FPB_TRY(check_plain_seq(o, dtype, B, T, H, dv, vb)); FPB_TRY(check_plain_seq(z, dtype, B, T, H, dv, vb));
  FPB_TRY(check_plain_seq(y, dtype, B, T, H, dv, vb));
  FPB_TRY(check_device());
  if ((int64_t)B * T * H == 0) return FPB_OK;
  const SeqView none{nullptr, 0, 0, 0};
  const bool wide = dv % 4 == 0 && check_plain_seq(o, dtype, B, T, H, dv, 2 * vb) == FPB_OK &&
                    check_plain_seq(z, dtype, B, T, H, dv, 2 * vb) == FPB_OK && check_plain_seq(y, dtype, B, T, H, dv, 2 * vb) == FPB_OK;
  const bool packed = check_plain_seq(o, dtype, B, T, H, dv, 16) == FPB_OK && check_plain_seq(z, dtype, B, T, H, dv, 16) == FPB_OK &&
                      check_plain_seq(y, dtype, B, T, H, dv, 16) == FPB_OK;
  launch_gn_gate(dtype, false, wide, packed, B, T, H, dv, eps, swish != 0, view(o), view(z), view(y), none, none, none, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_groupnorm_gate_bwd(int32_t B, int32_t T, int32_t H, int32_t dv, int32_t dtype, float eps, int32_t swish,
                           const fpb_seq* o, const fpb_seq* z, const fpb_seq* d_y, const fpb_seq* d_o, const fpb_seq* d_z,
                           fpb_stream_t stream) {
  if (B < 0 || T < 0 || H < 0 || dv <= 0 || dv % 2 || dv > 256) return FPB_ERR_BAD_SHAPE;
  if ((int64_t)B * T * H >= (1ll << 31)) return FPB_ERR_TOO_LARGE;
  if (!dtype_ok(dtype)) return FPB_ERR_BAD_DTYPE;
  const int vb = dtype == FPB_F32 ? 8 : 4;
  FPB_TRY(check_plain_seq(o, dtype, B, T, H, dv, vb)); FPB_TRY(check_plain_seq(z, dtype, B, T, H, dv, vb));
  FPB_TRY(check_plain_seq(d_y, dtype, B, T, H, dv, vb)); FPB_TRY(check_plain_seq(d_o, dtype, B, T, H, dv, vb));
  FPB_TRY(check_plain_seq(d_z, dtype, B, T, H, dv, vb));
  FPB_TRY(check_device());
  if ((int64_t)B * T * H == 0) return FPB_OK;
  const SeqView none{nullptr, 0, 0, 0};
  bool wide = dv % 4 == 0;
  for (const fpb_seq* s : {o, z, d_y, d_o, d_z}) wide = wide && check_plain_seq(s, dtype, B, T, H, dv, 2 * vb) == FPB_OK;
  bool packed = true;
  for (const fpb_seq* s : {o, z, d_y, d_o, d_z}) packed = packed && check_plain_seq(s, dtype, B, T, H, dv, 16) == FPB_OK;
  launch_gn_gate(dtype, true, wide, packed, B, T, H, dv, eps, swish != 0, view(o), view(z), none, view(d_y), view(d_o), view(d_z), (cudaStream_t)stream);
  return finish_launches(1, -1);
}

namespace {
int check_norm(int64_t rows, int32_t d, int32_t dtype, const void* a, int64_t a_stride, const void* b, int64_t b_stride) {
  if (rows < 0 || d <= 0) return FPB_ERR_BAD_SHAPE;
  if (!dtype_ok(dtype)) return FPB_ERR_BAD_DTYPE;
  const int vec = dtype == FPB_F32 ? 4 : 8;
  if (d % vec || d > 4 * 32 * vec) return FPB_ERR_BAD_SHAPE;
  if (rows == 0) return FPB_OK;
  if (!a || !b) return FPB_ERR_NULL_POINTER;
  if ((rows > 1 && (a_stride < d || b_stride < d)) || a_stride % vec || b_stride % vec || (uintptr_t)a % 16 || (uintptr_t)b % 16)
    return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}
}  // namespace

int fpb_layernorm_fwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride,
                      const float* weight, const float* bias, void* y, int64_t y_stride, fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, x, x_stride, y, y_stride));
  if ((uintptr_t)weight % 16 || (uintptr_t)bias % 16) return FPB_ERR_BAD_STRIDE;
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  launch_layernorm(dtype, false, rows, d, eps, x, x_stride, weight, bias, y, y_stride, nullptr, nullptr, nullptr, nullptr,
                   (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_layernorm_bwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride,
                      const float* weight, const void* d_y, int64_t dy_stride, void* d_x, float* d_weight, float* d_bias,
                      fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, x, x_stride, d_y, dy_stride));
  if (rows > 0 && (!d_x || (uintptr_t)d_x % 16)) return d_x ? FPB_ERR_BAD_STRIDE : FPB_ERR_NULL_POINTER;
  if ((uintptr_t)weight % 16) return FPB_ERR_BAD_STRIDE;
  FPB_TRY(check_device());
  // the kernel adds its partial sums into the two gradient vectors
  if (d_weight && cudaMemsetAsync(d_weight, 0, sizeof(float) * d, (cudaStream_t)stream) != cudaSuccess) return finish_launches(0, -1);
  if (d_bias && cudaMemsetAsync(d_bias, 0, sizeof(float) * d, (cudaStream_t)stream) != cudaSuccess) return finish_launches(0, -1);
  if (rows == 0) return FPB_OK;
  launch_layernorm(dtype, true, rows, d, eps, x, x_stride, weight, nullptr, nullptr, dy_stride, d_y, d_x, d_weight, d_bias,
                   (cudaStream_t)stream);
  return finish_launches(1, -1);
}

namespace {
// a (mod_rows, d) operand shared by rows_per_mod consecutive rows of the activations
int check_mod(int64_t rows, int32_t d, int32_t dtype, const void* ptr, int64_t mod_stride, int64_t rows_per_mod) {
  if (rows_per_mod <= 0) return FPB_ERR_BAD_SHAPE;
  if (rows == 0) return FPB_OK;
  if (!ptr) return FPB_ERR_NULL_POINTER;
  const int vec = dtype == FPB_F32 ? 4 : 8;
  const int64_t mod_rows = (rows + rows_per_mod - 1) / rows_per_mod;
  if ((mod_rows > 1 && mod_stride < d) || mod_stride % vec || (uintptr_t)ptr % 16) return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}
}  // namespace

int fpb_adaln_fwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride, const void* shift,
                  const void* scale, int64_t mod_stride, int64_t rows_per_mod, void* y, int64_t y_stride, fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, x, x_stride, y, y_stride));
  FPB_TRY(check_mod(rows, d, dtype, shift, mod_stride, rows_per_mod)); FPB_TRY(check_mod(rows, d, dtype, scale, mod_stride, rows_per_mod));
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  launch_adaln(dtype, false, rows, d, eps, x, x_stride, shift, scale, mod_stride, rows_per_mod, y, y_stride, nullptr, 0, nullptr,
               nullptr, nullptr, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_adaln_bwd(int64_t rows, int32_t d, int32_t dtype, float eps, const void* x, int64_t x_stride, const void* scale,
                  int64_t mod_stride, int64_t rows_per_mod, const void* d_y, int64_t dy_stride, void* d_x, float* d_shift,
                  float* d_scale, fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, x, x_stride, d_y, dy_stride));
  FPB_TRY(check_mod(rows, d, dtype, scale, mod_stride, rows_per_mod));
  if (rows > 0 && (!d_x || !d_shift || !d_scale)) return FPB_ERR_NULL_POINTER;
  if ((uintptr_t)d_x % 16) return FPB_ERR_BAD_STRIDE;
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  // the kernel adds its partial sums into the two gradient matrices
  const size_t gbytes = (size_t)((rows + rows_per_mod - 1) / rows_per_mod) * d * sizeof(float);
  if (cudaMemsetAsync(d_shift, 0, gbytes, (cudaStream_t)stream) != cudaSuccess ||
      cudaMemsetAsync(d_scale, 0, gbytes, (cudaStream_t)stream) != cudaSuccess)
    return finish_launches(0, -1);
  launch_adaln(dtype, true, rows, d, eps, x, x_stride, nullptr, scale, mod_stride, rows_per_mod, nullptr, 0, d_y, dy_stride, d_x,
               d_shift, d_scale, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_gate_residual_fwd(int64_t rows, int32_t d, int32_t dtype, const void* x, int64_t x_stride, const void* branch,
                          int64_t branch_stride, const void* gate, int64_t mod_stride, int64_t rows_per_mod, void* out,
                          int64_t out_stride, fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, x, x_stride, out, out_stride));
  FPB_TRY(check_norm(rows, d, dtype, branch, branch_stride, out, out_stride));
  FPB_TRY(check_mod(rows, d, dtype, gate, mod_stride, rows_per_mod));
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  launch_gate_residual(dtype, false, rows, d, x, x_stride, branch, branch_stride, gate, mod_stride, rows_per_mod, out, out_stride,
                       nullptr, nullptr, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_gate_residual_bwd(int64_t rows, int32_t d, int32_t dtype, const void* branch, int64_t branch_stride, const void* gate,
                          int64_t mod_stride, int64_t rows_per_mod, const void* d_out, int64_t dout_stride, void* d_branch,
                          float* d_gate, fpb_stream_t stream) {
  FPB_TRY(check_norm(rows, d, dtype, branch, branch_stride, d_out, dout_stride));
  FPB_TRY(check_mod(rows, d, dtype, gate, mod_stride, rows_per_mod));
  if (rows > 0 && (!d_branch || !d_gate)) return FPB_ERR_NULL_POINTER;
  if ((uintptr_t)d_branch % 16) return FPB_ERR_BAD_STRIDE;
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  const size_t gbytes = (size_t)((rows + rows_per_mod - 1) / rows_per_mod) * d * sizeof(float);
  if (cudaMemsetAsync(d_gate, 0, gbytes, (cudaStream_t)stream) != cudaSuccess) return finish_launches(0, -1);
  launch_gate_residual(dtype, true, rows, d, d_out, dout_stride, branch, branch_stride, gate, mod_stride, rows_per_mod, nullptr, 0,
                       d_branch, d_gate, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

namespace {
int check_xent(int64_t rows, int32_t V, int32_t dtype, const void* logits, int64_t row_stride) {
  if (rows < 0 || V <= 0) return FPB_ERR_BAD_SHAPE;
  if (rows >= (1ll << 31)) return FPB_ERR_TOO_LARGE;
  if (!dtype_ok(dtype)) return FPB_ERR_BAD_DTYPE;
  if (rows == 0) return FPB_OK;
  if (!logits) return FPB_ERR_NULL_POINTER;
  const int vec = dtype == FPB_F32 ? 4 : 8;
  if ((rows > 1 && row_stride < V) || row_stride % vec || (uintptr_t)logits % 16) return FPB_ERR_BAD_STRIDE;
  return FPB_OK;
}
}  // namespace

int fpb_cross_entropy_fwd(int64_t rows, int32_t V, int32_t dtype, const void* logits, int64_t row_stride, const int64_t* targets,
                          float* loss, float* lse, fpb_stream_t stream) {
  FPB_TRY(check_xent(rows, V, dtype, logits, row_stride));
  if (rows > 0 && (!targets || !loss || !lse)) return FPB_ERR_NULL_POINTER;
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  launch_xent_fwd(dtype, rows, V, logits, row_stride, targets, loss, lse, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

int fpb_cross_entropy_bwd(int64_t rows, int32_t V, int32_t dtype, const void* logits, int64_t row_stride, const int64_t* targets,
                          const float* lse, const float* scale, float row_weight, void* d_logits, int64_t d_stride,
                          fpb_stream_t stream) {
  FPB_TRY(check_xent(rows, V, dtype, logits, row_stride));
  FPB_TRY(check_xent(rows, V, dtype, d_logits, d_stride));
  if (rows > 0 && (!targets || !lse || !scale)) return FPB_ERR_NULL_POINTER;
  FPB_TRY(check_device());
  if (rows == 0) return FPB_OK;
  launch_xent_bwd(dtype, rows, V, logits, row_stride, targets, lse, scale, row_weight, d_logits, d_stride, (cudaStream_t)stream);
  return finish_launches(1, -1);
}

const char* fpb_strerror(int status) {
  switch (status) {
    case FPB_OK: return "ok";
    case FPB_ERR_NULL_POINTER: return "a required pointer is null";
    case FPB_ERR_BAD_SHAPE: return "unsupported or inconsistent shape (need 0 < dk, dv <= 256, H <= 256)";
    case FPB_ERR_BAD_DTYPE: return "unsupported dtype (bf16 and fp32 only)";
    case FPB_ERR_BAD_STRIDE: return "bad stride (inner stride must be 1, others positive and non-overlapping)";
    case FPB_ERR_BAD_DECAY: return "head decay outside [0, 1] or not finite";
    case FPB_ERR_BAD_BLOCK_SIZE: return "block_size must be positive";
    case FPB_ERR_NO_DEVICE_CODE: return "current CUDA device is not sm_100 (B200); this library has no other code path";
    case FPB_ERR_LAUNCH: return "CUDA launch failed (see fpb_last_cuda_error)";
    case FPB_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case FPB_ERR_TENSOR_MAP: return "could not encode a TMA tensor map for a tensor";
    case FPB_ERR_TOO_LARGE: return "size beyond a fixed limit of this entry point (batch over 65535, or more scratch than the built-in array holds)";
    case FPB_ERR_BAD_WORKSPACE: return "workspace pointer not 16-byte aligned or negative size";
    default: return "unknown status";
  }
}

int fpb_version(void) { return 200; }

int64_t fpb_workspace_bytes(const fpb_dims* dims) {
  // what lets the emptiest pass of this shape (one CTA per batch row and head) split as far as it would
  if (!dims || dims->B <= 0 || dims->H <= 0 || dims->T <= 0 || dims->dk <= 0 || dims->dv <= 0) return 0;
  if (dims->dtype != FPB_BF16 || check_device() != FPB_OK) return 0;
  // (the small state tiles run two CTAs per SM: ask for what that residency can use)
  const int ctas_per_sm = (dims->dk <= 64 || dims->dv <= 64) ? 2 : 1;
  const Segments sg = choose_segments((long long)dims->B * dims->H, ctas_per_sm, dims->T, 64, (long long)dims->B * dims->H,
                                      (long long)dims->dk * dims->dv, 0, dims->B);
  return sg.n > 1 ? (int64_t)dims->B * dims->H * sg.n * dims->dk * dims->dv * 4 : 0;
}
int fpb_last_path(void) { return tl_last_path; }
int fpb_last_cuda_error(void) { return tl_last_cuda_error; }
int64_t fpb_launch_count(void) { return g_launches.load(); }

int fpb_device_status(fpb_stream_t stream, int32_t* detail) {
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) { tl_last_cuda_error = (int)cudaGetLastError(); return FPB_ERR_LAUNCH; }
  int32_t word = 0;
  if (cudaMemcpyFromSymbol(&word, g_device_status, sizeof(word)) != cudaSuccess) { tl_last_cuda_error = (int)cudaGetLastError(); return FPB_ERR_LAUNCH; }
  if (detail) *detail = word;
  if (word == 0) return FPB_OK;
  const int32_t zero = 0;
  cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  return FPB_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
