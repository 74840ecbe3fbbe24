// PyTorch operator layer of the B200 KANLinear path: the compiled module `torchsplinekan_b200._C`.
//
// Counterpart of the reference's extension boundary (csrc/kan_ext.cpp: TORCH_LIBRARY(spline_kan) with
// CUDA and Meta kernels plus the pybind module `spline_kan._C`; csrc/kan_autograd.cpp: KANFunction and
// kan_apply; csrc/kan_ops.h: kan_check_inputs).  Same names, argument order, schemas and error
// behaviour.  Everything numerical happens in libkan_b200.so behind the C ABI of include/kan_b200.h:
// this file only validates, allocates outputs and scratch through PyTorch's caching allocator, passes
// raw pointers and the current stream, and keeps the autograd bookkeeping.  There is no CPU kernel:
// CPU tensors are rejected.
#include <torch/extension.h>
#include <torch/library.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/kan_b200.h"

namespace {

using at::Tensor;
namespace py = pybind11;

// ------------------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------------------
inline bool has(const Tensor& t) { return t.defined() && t.numel() > 0; }
inline const void* cptr(const Tensor& t) { return has(t) ? t.data_ptr() : nullptr; }
inline void* mptr(Tensor& t) { return has(t) ? t.data_ptr() : nullptr; }

inline int dtype_code(const Tensor& t) {
    if (t.scalar_type() == at::kFloat) return KANB200_F32;
    if (t.scalar_type() == at::kDouble) return KANB200_F64;
    TORCH_CHECK(false, "only FP32 and FP64 inputs are supported, got ", t.scalar_type());
}

void check_rc(int rc) {
    if (rc == KANB200_OK) return;
    const std::string msg = kanb200_last_error();
    if (rc == KANB200_EINVAL) TORCH_CHECK(false, msg);
    TORCH_CHECK(false, "kan_b200 error ", rc, ": ", msg);
}

std::atomic<int> g_mode{KANB200_MODE_AUTO};

int mode_from_name(const std::string& name) {
    if (name == "auto") return KANB200_MODE_AUTO;
    if (name == "simt") return KANB200_MODE_SIMT;
    if (name == "bf16x3") return KANB200_MODE_TC_BF16X3;
    if (name == "bf16x1") return KANB200_MODE_TC_BF16X1;
    return -1;
}
const char* mode_name(int m) {
    switch (m) {
        case KANB200_MODE_SIMT: return "simt";
        case KANB200_MODE_TC_BF16X3: return "bf16x3";
        case KANB200_MODE_TC_BF16X1: return "bf16x1";
        default: return "auto";
    }
}

// ------------------------------------------------------------------------------------------------
// scratch memory: one buffer per (device, stream, purpose), grown on demand, from the caching
// allocator.  The first word of a buffer is the sticky status word of the tensor-core kernels; the
// header also carries a pointer to one int of mapped pinned host memory that a reporting kernel sets
// as well, and every later call on the same buffer looks at that int without synchronising.
// ------------------------------------------------------------------------------------------------
enum Purpose { WS_FWD = 0, WS_BWD = 1, WS_BASIS = 2, WS_EDGE = 3, WS_EDGE_X = 4 };

struct Scratch {
    Tensor buf;
    int* mirror = nullptr;       // mapped pinned host int that a reporting kernel sets
    void* mirror_dev = nullptr;  // its device address, stored at byte 8 of the buffer's header
};

std::mutex g_ws_mutex;
std::map<std::tuple<int, int64_t, int>, Scratch> g_ws;

// True when the pinned copy of the status word shows that an earlier kernel on this buffer gave up
// a bounded wait; the pinned copy is reset (the device word is cleared by the caller's check).
bool reported(Scratch& s) {
    if (s.mirror && *reinterpret_cast<volatile int*>(s.mirror) != 0) {
        *s.mirror = 0;
        return true;
    }
    return false;
}

// Never throws while the registry lock is held: a pending report comes back in `pending`.
Scratch* scratch(const c10::Device& dev, cudaStream_t st, int purpose, size_t bytes) {
    if (bytes == 0) return nullptr;
    Scratch* out = nullptr;
    bool pending = false;
    void* old_buf = nullptr;
    Tensor keep_alive;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        auto key = std::make_tuple((int)dev.index(), (int64_t)reinterpret_cast<intptr_t>(st), purpose);
        Scratch& s = g_ws[key];
        if (s.buf.defined()) pending = reported(s);
        if (pending) {
            keep_alive = s.buf;
            old_buf = s.buf.data_ptr();
        }
        if (!s.buf.defined() || (size_t)s.buf.numel() < bytes) {
            s.buf = at::empty({(int64_t)bytes + 256}, at::TensorOptions().dtype(at::kByte).device(dev));
            C10_CUDA_CHECK(cudaMemsetAsync(s.buf.data_ptr(), 0, 256, st));
            // Host allocations and copies from pageable memory are not allowed while the stream is
            // being captured into a graph: a buffer first created there gets no host-visible int
            // (its device word still works, check_status reads it).
            cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
            C10_CUDA_CHECK(cudaStreamIsCapturing(st, &capturing));
            if (capturing == cudaStreamCaptureStatusNone) {
                if (!s.mirror) {
                    C10_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&s.mirror), sizeof(int), cudaHostAllocMapped));
                    *s.mirror = 0;
                }
                void* mirror_dev = nullptr;
                C10_CUDA_CHECK(cudaHostGetDevicePointer(&mirror_dev, s.mirror, 0));
                s.mirror_dev = mirror_dev;
                // the 8-byte source of this copy must outlive the call: it lives in the registry entry
                C10_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(s.buf.data_ptr()) + 8, &s.mirror_dev,
                                               sizeof(void*), cudaMemcpyHostToDevice, st));
            }
        }
        out = &s;
    }
    if (pending) {
        kanb200_check_status(old_buf, st);          // synchronises and clears the device word
        TORCH_CHECK(false, "kan_b200: an earlier tensor-core kernel on this stream gave up a bounded wait "
                           "(its outputs are incomplete); the status has been cleared");
    }
    return out;
}

void check_status_all() {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    for (auto& kv : g_ws) {
        Scratch& s = kv.second;
        if (!s.buf.defined()) continue;
        c10::cuda::CUDAGuard guard(s.buf.device());
        cudaStream_t st = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(std::get<1>(kv.first)));
        if (s.mirror) *s.mirror = 0;
        check_rc(kanb200_check_status(s.buf.data_ptr(), st));
    }
}

void release_workspaces() {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    for (auto& kv : g_ws)
        if (kv.second.mirror) cudaFreeHost(kv.second.mirror);
    g_ws.clear();
}

// Test hook: presets the status word of the (current device, current stream, purpose) buffer, and with
// `as_kernel` also the host-visible int, as a reporting kernel would.
void poke_status(int purpose, int code, bool as_kernel) {
    const auto dev = c10::Device(c10::kCUDA, (c10::DeviceIndex)at::cuda::current_device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = g_ws.find(std::make_tuple((int)dev.index(), (int64_t)reinterpret_cast<intptr_t>(st), purpose));
    TORCH_CHECK(it != g_ws.end() && it->second.buf.defined(), "no such workspace yet");
    C10_CUDA_CHECK(cudaMemcpyAsync(it->second.buf.data_ptr(), &code, sizeof(int), cudaMemcpyHostToDevice, st));
    C10_CUDA_CHECK(cudaStreamSynchronize(st));
    if (as_kernel && it->second.mirror) *it->second.mirror = code;
}

// Debugging aid (environment variable KAN_B200_BACKTRACE): native frames on a fatal signal.
void backtrace_on_signal(int sig) {
    void* frames[64];
    const int n = backtrace(frames, 64);
    const char msg[] = "kan_b200: fatal signal, native frames:\n";
    if (write(2, msg, sizeof(msg) - 1) < 0) {}
    backtrace_symbols_fd(frames, n, 2);
    signal(sig, SIG_DFL);
    raise(sig);
}
void install_backtrace_handler() {
    signal(SIGSEGV, backtrace_on_signal);
    signal(SIGFPE, backtrace_on_signal);
    signal(SIGABRT, backtrace_on_signal);
}

// ------------------------------------------------------------------------------------------------
// optional per-call timing (CUDA events on the launching stream), for the benchmark's roofline
// ------------------------------------------------------------------------------------------------
struct TimedCall {
    std::string name;
    cudaEvent_t a, b;
};
std::mutex g_ev_mutex;
bool g_ev_on = false;
std::vector<TimedCall> g_events;

struct ScopedTimer {
    bool on;
    TimedCall t;
    cudaStream_t st;
    ScopedTimer(const char* name, cudaStream_t s) : on(g_ev_on), st(s) {
        if (!on) return;
        t.name = name;
        cudaEventCreate(&t.a);
        cudaEventCreate(&t.b);
        cudaEventRecord(t.a, st);
    }
    ~ScopedTimer() {
        if (!on) return;
        cudaEventRecord(t.b, st);
        std::lock_guard<std::mutex> lock(g_ev_mutex);
        g_events.push_back(t);
    }
};

void set_event_log(bool on) {
    std::lock_guard<std::mutex> lock(g_ev_mutex);
    g_ev_on = on;
}

std::vector<std::pair<std::string, double>> take_event_log() {
    std::vector<TimedCall> ev;
    {
        std::lock_guard<std::mutex> lock(g_ev_mutex);
        ev.swap(g_events);
    }
    std::vector<std::pair<std::string, double>> out;
    for (auto& t : ev) {
        cudaEventSynchronize(t.b);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, t.a, t.b);
        out.emplace_back(t.name, (double)ms);
        cudaEventDestroy(t.a);
        cudaEventDestroy(t.b);
    }
    return out;
}

// ------------------------------------------------------------------------------------------------
// validation before any launch (kan_check_inputs, csrc/kan_ops.h:27-78)
// ------------------------------------------------------------------------------------------------
struct Dims {
    int64_t N, I, O;
    int G, k;
};

Dims check_inputs(const Tensor& x, const Tensor& grid, const Tensor& base_weight, const Tensor& spline_weight,
                  const Tensor& spline_scaler, int64_t spline_order, bool has_scaler) {
    TORCH_CHECK(x.dim() == 2, "x must be 2-D [B, I], got ", x.dim(), "-D");
    TORCH_CHECK(grid.dim() == 2, "grid must be 2-D [I, G+2k+1]");
    TORCH_CHECK(spline_weight.dim() == 3, "spline_weight must be 3-D [O, I, R]");
    TORCH_CHECK(spline_order >= 1 && spline_order <= 3, "spline_order must be 1, 2 or 3; got ", spline_order);
    const int64_t I = x.size(1), O = spline_weight.size(0), T = grid.size(1);
    const int64_t G = T - 2 * spline_order - 1;
    TORCH_CHECK(G >= 1, "grid has ", T, " knots, too few for spline_order ", spline_order);
    TORCH_CHECK(grid.size(0) == I, "grid.size(0)=", grid.size(0), " must equal in_features=", I);
    TORCH_CHECK(spline_weight.size(1) == I, "spline_weight.size(1) must equal in_features=", I);
    TORCH_CHECK(spline_weight.size(2) == G + spline_order, "spline_weight.size(2)=", spline_weight.size(2),
                " but grid implies R=G+k=", G + spline_order);
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kDouble,
                "only FP32 and FP64 inputs are supported, got ", x.scalar_type());
    TORCH_CHECK(grid.scalar_type() == x.scalar_type() && spline_weight.scalar_type() == x.scalar_type(),
                "x, grid and spline_weight must share a dtype");
    TORCH_CHECK(grid.device() == x.device() && spline_weight.device() == x.device(),
                "x, grid and spline_weight must be on the same device");
    if (has(base_weight)) {
        TORCH_CHECK(base_weight.dim() == 2 && base_weight.size(0) == O && base_weight.size(1) == I,
                    "base_weight must have shape [O, I] = [", O, ", ", I, "]");
        TORCH_CHECK(base_weight.scalar_type() == x.scalar_type() && base_weight.device() == x.device(),
                    "base_weight must match x in dtype and device");
    }
    if (has_scaler) {
        TORCH_CHECK(spline_scaler.defined() && spline_scaler.dim() == 2 && spline_scaler.size(0) == O &&
                        spline_scaler.size(1) == I,
                    "spline_scaler must have shape [O, I] = [", O, ", ", I, "]");
        TORCH_CHECK(spline_scaler.scalar_type() == x.scalar_type() && spline_scaler.device() == x.device(),
                    "spline_scaler must match x in dtype and device");
    }
    TORCH_CHECK(x.is_cuda(), "kan_b200: x must be a CUDA tensor (this backend has no CPU kernels)");
    TORCH_CHECK(G + 2 * spline_order <= KANB200_MAX_DEG0_BASIS, "CUDA kernel supports G + 2k <= ",
                KANB200_MAX_DEG0_BASIS, " (got G=", G, ", k=", spline_order,
                "); use backend='reference' for larger grids");
    TORCH_CHECK(I <= KANB200_MAX_IN_FEATURES, "CUDA kernel supports in_features <= ", KANB200_MAX_IN_FEATURES,
                ", got ", I);
    return Dims{x.size(0), I, O, (int)G, (int)spline_order};
}

inline Tensor contig_or_absent(const Tensor& t) { return has(t) ? t.contiguous() : Tensor(); }

// ------------------------------------------------------------------------------------------------
// forward / backward through the C ABI
// ------------------------------------------------------------------------------------------------
Tensor forward_impl(const Tensor& x, const Tensor& grid, const Tensor& base_weight, const Tensor& spline_weight,
                    const Tensor& spline_scaler, int64_t spline_order, bool has_scaler) {
    const Dims d = check_inputs(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler);
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    Tensor y = at::empty({d.N, d.O}, x.options());
    if (d.N == 0) return y;
    const Tensor xc = x.contiguous(), gc = grid.contiguous(), bw = contig_or_absent(base_weight),
                 sw = spline_weight.contiguous(), sc = has_scaler ? contig_or_absent(spline_scaler) : Tensor();
    const int code = dtype_code(x), mode = g_mode.load();
    const size_t bytes = kanb200_workspace_bytes(KANB200_OP_FORWARD, mode, code, d.N, d.I, d.O, d.G, d.k, 1, 1);
    Scratch* ws = scratch(x.device(), st, WS_FWD, bytes);
    {
        ScopedTimer timer("forward", st);
        check_rc(kanb200_forward(code, mode, xc.data_ptr(), gc.data_ptr(), cptr(bw), sw.data_ptr(), cptr(sc),
                                 y.data_ptr(), d.N, d.I, d.O, d.G, d.k, ws ? ws->buf.data_ptr() : nullptr,
                                 ws ? (size_t)ws->buf.numel() : 0, st));
    }
    return y;
}

// Inference with fixed parameters: table + weight image built once (prepare_forward), contraction
// alone per call (forward_prepared).  An empty result of prepare_forward means "no prepared form".
Tensor prepare_forward(const Tensor& grid, const Tensor& base_weight, const Tensor& spline_weight,
                       const Tensor& spline_scaler, int64_t spline_order, bool has_scaler) {
    TORCH_CHECK(spline_weight.is_cuda() && spline_weight.dim() == 3, "prepare_forward: spline_weight must be a CUDA "
                "tensor [O, I, G+k]");
    TORCH_CHECK(grid.is_cuda() && grid.dim() == 2, "prepare_forward: grid must be a CUDA tensor [I, G+2k+1]");
    const int64_t O = spline_weight.size(0), I = spline_weight.size(1);
    const int64_t G = grid.size(1) - 2 * spline_order - 1;
    TORCH_CHECK(grid.size(0) == I && spline_weight.size(2) == G + spline_order, "prepare_forward: shapes do not agree");
    const bool has_base = has(base_weight);
    const int code = dtype_code(spline_weight);
    const size_t bytes = kanb200_prepared_bytes(code, I, O, (int)G, (int)spline_order, has_base ? 1 : 0);
    Tensor buf = at::empty({(int64_t)bytes}, spline_weight.options().dtype(at::kByte));
    if (bytes == 0) return buf;
    c10::cuda::CUDAGuard guard(spline_weight.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const Tensor gc = grid.contiguous(), bw = contig_or_absent(base_weight), sw = spline_weight.contiguous(),
                 sc = has_scaler ? contig_or_absent(spline_scaler) : Tensor();
    check_rc(kanb200_prepare_forward(code, gc.data_ptr(), cptr(bw), sw.data_ptr(), cptr(sc), I, O, (int)G,
                                     (int)spline_order, buf.data_ptr(), bytes, st));
    return buf;
}

Tensor forward_prepared(const Tensor& x, const Tensor& prepared, int64_t O, int64_t G, int64_t spline_order,
                        bool has_base) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kFloat,
                "forward_prepared: x must be a float32 CUDA tensor [B, I]");
    TORCH_CHECK(prepared.is_cuda() && prepared.scalar_type() == at::kByte && prepared.is_contiguous() &&
                    prepared.device() == x.device(),
                "forward_prepared: prepared must be the buffer of prepare_forward on x's device");
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = x.size(0), I = x.size(1);
    Tensor y = at::empty({N, O}, x.options());
    if (N == 0) return y;
    const Tensor xc = x.contiguous();
    int mode = g_mode.load();
    if (mode == KANB200_MODE_SIMT) mode = KANB200_MODE_AUTO;     // the prepared form exists on the tensor cores only
    size_t bytes = kanb200_workspace_bytes(KANB200_OP_FORWARD, KANB200_MODE_TC_BF16X3, dtype_code(x), N, I, O, (int)G,
                                           (int)spline_order, 1, 1);
    Scratch* ws = scratch(x.device(), st, WS_FWD, bytes < 256 ? 256 : bytes);
    {
        ScopedTimer timer("forward", st);
        check_rc(kanb200_forward_prepared(dtype_code(x), mode, xc.data_ptr(), prepared.data_ptr(),
                                          (size_t)prepared.numel(), has_base ? 1 : 0, y.data_ptr(), N, I, O, (int)G,
                                          (int)spline_order, ws->buf.data_ptr(), (size_t)ws->buf.numel(), st));
    }
    return y;
}

struct Grads {
    Tensor gx, gb, gs, gc;
};

Grads backward_impl(const Tensor& grad_output, const Tensor& x, const Tensor& grid, const Tensor& base_weight,
                    const Tensor& spline_weight, const Tensor& spline_scaler, int64_t spline_order, bool has_scaler,
                    bool need_x, bool need_base, bool need_spline) {
    const Dims d = check_inputs(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler);
    TORCH_CHECK(grad_output.dim() == 2 && grad_output.size(0) == d.N && grad_output.size(1) == d.O,
                "grad_output must have shape [B, O]");
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const bool has_base = has(base_weight);
    need_base = need_base && has_base;
    const bool need_scaler = need_spline && has_scaler;
    Grads g;
    if (need_x) g.gx = at::empty_like(x, x.options(), at::MemoryFormat::Contiguous);
    if (need_base) g.gb = at::empty_like(base_weight, base_weight.options(), at::MemoryFormat::Contiguous);
    if (need_spline) g.gs = at::empty_like(spline_weight, spline_weight.options(), at::MemoryFormat::Contiguous);
    if (need_scaler) g.gc = at::empty_like(spline_scaler, spline_scaler.options(), at::MemoryFormat::Contiguous);
    const Tensor D = grad_output.to(x.scalar_type()).contiguous(), xc = x.contiguous(), gc = grid.contiguous(),
                 bw = contig_or_absent(base_weight), sw = spline_weight.contiguous(),
                 sc = has_scaler ? contig_or_absent(spline_scaler) : Tensor();
    const int code = dtype_code(x), mode = g_mode.load();
    const size_t bytes = kanb200_workspace_bytes(KANB200_OP_BACKWARD, mode, code, d.N, d.I, d.O, d.G, d.k,
                                                 need_x ? 1 : 0, (need_base || need_spline) ? 1 : 0);
    Scratch* ws = scratch(x.device(), st, WS_BWD, bytes);
    {
        ScopedTimer timer("backward", st);
        check_rc(kanb200_backward(code, mode, cptr(D), cptr(xc), gc.data_ptr(), cptr(bw), sw.data_ptr(), cptr(sc),
                                  mptr(g.gx), mptr(g.gb), mptr(g.gs), mptr(g.gc), d.N, d.I, d.O, d.G, d.k,
                                  ws ? ws->buf.data_ptr() : nullptr, ws ? (size_t)ws->buf.numel() : 0, st));
    }
    return g;
}

// ------------------------------------------------------------------------------------------------
// stand-alone basis operators (kan_basis_cuda / kan_basis_grad_cuda, csrc/kan_cuda.cu:666-699)
// ------------------------------------------------------------------------------------------------
int check_basis_args(const Tensor& x, const Tensor& grid, int64_t k) {
    TORCH_CHECK(x.is_cuda() && grid.is_cuda(), "kan_basis: x and grid must be CUDA tensors");
    TORCH_CHECK(x.dim() == 2 && grid.dim() == 2 && grid.size(0) == x.size(1),
                "kan_basis: x must be [B, I] and grid [I, G+2k+1]");
    TORCH_CHECK(k >= 1 && k <= 3, "kan_basis: spline_order must be 1, 2 or 3");
    TORCH_CHECK(x.scalar_type() == grid.scalar_type(), "kan_basis: dtype mismatch");
    TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kDouble, "kan_basis: only FP32/FP64 supported");
    const int64_t G = grid.size(1) - 2 * k - 1;
    TORCH_CHECK(G >= 1, "kan_basis: grid too short");
    TORCH_CHECK(G + 2 * k <= KANB200_MAX_DEG0_BASIS, "CUDA kernel supports G + 2k <= ", KANB200_MAX_DEG0_BASIS,
                " (got G=", G, ", k=", k, ")");
    TORCH_CHECK(x.size(1) <= KANB200_MAX_IN_FEATURES, "kan_basis: too many input features");
    return (int)G;
}

Tensor basis(const Tensor& x, const Tensor& grid, int64_t k) {
    const int G = check_basis_args(x, grid, k);
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = x.size(0), I = x.size(1);
    Tensor H = at::empty({N, I, G + k}, x.options());
    if (N == 0) return H;
    const Tensor xc = x.contiguous(), gc = grid.contiguous();
    const int code = dtype_code(x);
    Scratch* ws = scratch(x.device(), st, WS_BASIS,
                          kanb200_workspace_bytes(KANB200_OP_BASIS, KANB200_MODE_AUTO, code, N, I, 1, G, (int)k, 0, 0));
    check_rc(kanb200_basis_ws(code, xc.data_ptr(), gc.data_ptr(), H.data_ptr(), N, I, G, (int)k,
                              ws ? ws->buf.data_ptr() : nullptr, ws ? (size_t)ws->buf.numel() : 0, st));
    return H;
}

Tensor basis_grad(const Tensor& x, const Tensor& grid, int64_t k, const Tensor& grad_basis) {
    const int G = check_basis_args(x, grid, k);
    TORCH_CHECK(grad_basis.dim() == 3 && grad_basis.size(0) == x.size(0) && grad_basis.size(1) == x.size(1) &&
                    grad_basis.size(2) == G + k,
                "kan_basis_grad: gH must be [B, I, G+k]");
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = x.size(0), I = x.size(1);
    Tensor gx = at::empty({N, I}, x.options());
    if (N == 0) return gx;
    const Tensor xc = x.contiguous(), gc = grid.contiguous(), gH = grad_basis.to(x.scalar_type()).contiguous();
    const int code = dtype_code(x);
    Scratch* ws = scratch(x.device(), st, WS_BASIS,
                          kanb200_workspace_bytes(KANB200_OP_BASIS, KANB200_MODE_AUTO, code, N, I, 1, G, (int)k, 0, 0));
    check_rc(kanb200_basis_grad_ws(code, xc.data_ptr(), gc.data_ptr(), gH.data_ptr(), gx.data_ptr(), N, I, G, (int)k,
                                   ws ? ws->buf.data_ptr() : nullptr, ws ? (size_t)ws->buf.numel() : 0, st));
    return gx;
}

// ------------------------------------------------------------------------------------------------
// edge statistic (edge_abs_mean_cuda / edge_abs_mean_backward_cuda, csrc/kan_reg_cuda.cu:263-312)
// ------------------------------------------------------------------------------------------------
void check_edge(const Tensor& s, const Tensor& H, const Tensor& bw, const Tensor& W, bool has_base) {
    TORCH_CHECK(H.is_cuda() && W.is_cuda(), "edge_abs_mean: H and W must be CUDA tensors");
    TORCH_CHECK(H.dim() == 3 && W.dim() == 3, "edge_abs_mean: H must be [N,I,R], W [O,I,R]");
    TORCH_CHECK(H.size(1) == W.size(1) && H.size(2) == W.size(2), "edge_abs_mean: H/W shape mismatch");
    TORCH_CHECK(H.size(2) <= 72, "edge_abs_mean: R must be <= 72, got ", H.size(2));
    TORCH_CHECK(H.size(1) <= KANB200_MAX_IN_FEATURES, "edge_abs_mean: too many input features");
    TORCH_CHECK(H.size(0) >= 1, "edge_abs_mean: need at least one sample");
    TORCH_CHECK(H.scalar_type() == W.scalar_type(), "edge_abs_mean: dtype mismatch");
    TORCH_CHECK(H.scalar_type() == at::kFloat || H.scalar_type() == at::kDouble,
                "edge_abs_mean: only FP32/FP64 supported");
    if (has_base) {
        TORCH_CHECK(s.dim() == 2 && s.size(0) == H.size(0) && s.size(1) == H.size(1), "edge_abs_mean: s must be [N, I]");
        TORCH_CHECK(bw.dim() == 2 && bw.size(0) == W.size(0) && bw.size(1) == W.size(1),
                    "edge_abs_mean: base_weight must be [O, I]");
        TORCH_CHECK(s.scalar_type() == H.scalar_type() && bw.scalar_type() == H.scalar_type(),
                    "edge_abs_mean: dtype mismatch");
    }
}

Tensor edge_abs_mean(const Tensor& s, const Tensor& H, const Tensor& base_weight, const Tensor& W) {
    const bool has_base = has(base_weight);
    check_edge(s, H, base_weight, W, has_base);
    c10::cuda::CUDAGuard guard(H.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = H.size(0), I = H.size(1), R = H.size(2), O = W.size(0);
    Tensor a = at::empty({O, I}, H.options());
    const Tensor sc = has_base ? s.contiguous() : Tensor(), Hc = H.contiguous(),
                 bw = has_base ? base_weight.contiguous() : Tensor(), Wc = W.contiguous();
    const int code = dtype_code(H);
    Scratch* ws = scratch(H.device(), st, WS_EDGE,
                          kanb200_workspace_bytes(KANB200_OP_EDGE_FWD, KANB200_MODE_SIMT, code, N, I, O,
                                                  (int)std::max<int64_t>(R - 1, 1), 1, 0, 0));
    check_rc(kanb200_edge_abs_mean(code, cptr(sc), Hc.data_ptr(), cptr(bw), Wc.data_ptr(), a.data_ptr(), N, I, O,
                                   (int)R, ws ? ws->buf.data_ptr() : nullptr, ws ? (size_t)ws->buf.numel() : 0, st));
    return a;
}

std::tuple<Tensor, Tensor, Tensor, Tensor> edge_abs_mean_backward(const Tensor& grad_a, const Tensor& s, const Tensor& H,
                                                                  const Tensor& base_weight, const Tensor& W,
                                                                  bool need_s, bool need_H, bool need_bw, bool need_W) {
    const bool has_base = has(base_weight);
    check_edge(s, H, base_weight, W, has_base);
    TORCH_CHECK(grad_a.dim() == 2 && grad_a.size(0) == W.size(0) && grad_a.size(1) == W.size(1),
                "edge_abs_mean_backward: grad shape");
    c10::cuda::CUDAGuard guard(H.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = H.size(0), I = H.size(1), R = H.size(2), O = W.size(0);
    Tensor ds, dH, dbw, dW;
    if (need_s && has_base) ds = at::empty({N, I}, H.options());
    if (need_H) dH = at::empty({N, I, R}, H.options());
    if (need_bw && has_base) dbw = at::empty({O, I}, H.options());
    if (need_W) dW = at::empty({O, I, R}, H.options());
    const Tensor ga = grad_a.to(W.scalar_type()).contiguous(), sc = has_base ? s.contiguous() : Tensor(),
                 Hc = H.contiguous(), bw = has_base ? base_weight.contiguous() : Tensor(), Wc = W.contiguous();
    const int code = dtype_code(H);
    Scratch* ws = scratch(H.device(), st, WS_EDGE,
                          kanb200_workspace_bytes(KANB200_OP_EDGE_BWD, KANB200_MODE_SIMT, code, N, I, O,
                                                  (int)std::max<int64_t>(R - 1, 1), 1, 0, 0));
    check_rc(kanb200_edge_abs_mean_backward(code, ga.data_ptr(), cptr(sc), Hc.data_ptr(), cptr(bw), Wc.data_ptr(),
                                            mptr(ds), mptr(dH), mptr(dbw), mptr(dW), N, I, O, (int)R,
                                            ws ? ws->buf.data_ptr() : nullptr, ws ? (size_t)ws->buf.numel() : 0, st));
    return std::make_tuple(ds, dH, dbw, dW);
}

// ------------------------------------------------------------------------------------------------
// edge statistic straight from the layer input (no counterpart among the reference's operators:
// it fuses kan_basis_cuda + edge_abs_mean_cuda, and in backward edge_abs_mean_backward_cuda +
// kan_basis_grad_cuda, so that H [N,I,R] and dH never exist).  s: the caller's base values [N,I],
// or an empty tensor = silu(x); base_weight empty = no base term; W = effective coefficients.
// ------------------------------------------------------------------------------------------------
int check_edge_x(const Tensor& x, const Tensor& s, const Tensor& grid, const Tensor& bw, const Tensor& W, int64_t k) {
    const int G = check_basis_args(x, grid, k);
    TORCH_CHECK(W.is_cuda() && W.dim() == 3 && W.size(1) == x.size(1) && W.size(2) == G + k,
                "edge_abs_mean_x: W must be a CUDA tensor [O, I, G+k]");
    TORCH_CHECK(W.scalar_type() == x.scalar_type(), "edge_abs_mean_x: dtype mismatch");
    TORCH_CHECK(x.size(0) >= 1, "edge_abs_mean: need at least one sample");
    if (has(bw))
        TORCH_CHECK(bw.dim() == 2 && bw.size(0) == W.size(0) && bw.size(1) == W.size(1) &&
                        bw.scalar_type() == x.scalar_type(),
                    "edge_abs_mean_x: base_weight must be [O, I]");
    if (has(s))
        TORCH_CHECK(has(bw) && s.dim() == 2 && s.size(0) == x.size(0) && s.size(1) == x.size(1) &&
                        s.scalar_type() == x.scalar_type(),
                    "edge_abs_mean_x: s must be [N, I] and needs base_weight");
    return G;
}

Tensor edge_abs_mean_x(const Tensor& x, const Tensor& s, const Tensor& grid, const Tensor& base_weight, const Tensor& W,
                       int64_t k) {
    const int G = check_edge_x(x, s, grid, base_weight, W, k);
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = x.size(0), I = x.size(1), O = W.size(0);
    Tensor a = at::empty({O, I}, x.options());
    const Tensor xc = x.contiguous(), sc = contig_or_absent(s), gc = grid.contiguous(),
                 bw = contig_or_absent(base_weight), Wc = W.contiguous();
    const int code = dtype_code(x), mode = g_mode.load();
    Scratch* ws = scratch(x.device(), st, WS_EDGE_X,
                          kanb200_workspace_bytes(KANB200_OP_EDGE_X_FWD, mode, code, N, I, O, G, (int)k, 0, 0));
    {
        ScopedTimer timer("edge_forward", st);
        check_rc(kanb200_edge_abs_mean_x(code, mode, xc.data_ptr(), cptr(sc), gc.data_ptr(), cptr(bw), Wc.data_ptr(),
                                         a.data_ptr(), N, I, O, G, (int)k, ws ? ws->buf.data_ptr() : nullptr,
                                         ws ? (size_t)ws->buf.numel() : 0, st));
    }
    return a;
}

// Scalar head of the activation regulariser and its gradient with respect to the edge statistic, in one
// launch (kanb200_edge_penalty).
std::tuple<Tensor, Tensor> edge_penalty(const Tensor& a, double mu1, double mu2) {
    TORCH_CHECK(a.is_cuda() && a.numel() > 0, "edge_penalty: a must be a non-empty CUDA tensor");
    c10::cuda::CUDAGuard guard(a.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const Tensor ac = a.contiguous();
    Tensor value = at::empty({}, a.options()), grad = at::empty_like(ac);
    const size_t ws_bytes = kanb200_edge_penalty_workspace_bytes();
    Tensor ws = at::empty({(int64_t)ws_bytes}, a.options().dtype(at::kByte));
    check_rc(kanb200_edge_penalty(dtype_code(a), ac.data_ptr(), ac.numel(), mu1, mu2, value.data_ptr(),
                                  grad.data_ptr(), ws.data_ptr(), ws_bytes, st));
    return {value, grad.view(a.sizes())};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> edge_abs_mean_x_backward(const Tensor& grad_a, const Tensor& x, const Tensor& s,
                                                                    const Tensor& grid, const Tensor& base_weight,
                                                                    const Tensor& W, int64_t k, bool need_x, bool need_s,
                                                                    bool need_bw, bool need_W) {
    const int G = check_edge_x(x, s, grid, base_weight, W, k);
    TORCH_CHECK(grad_a.dim() == 2 && grad_a.size(0) == W.size(0) && grad_a.size(1) == W.size(1),
                "edge_abs_mean_x_backward: grad shape");
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int64_t N = x.size(0), I = x.size(1), O = W.size(0), R = W.size(2);
    const bool has_base = has(base_weight);
    Tensor gx, ds, dbw, dW;
    if (need_x) gx = at::empty({N, I}, x.options());
    if (need_s && has_base && has(s)) ds = at::empty({N, I}, x.options());
    if (need_bw && has_base) dbw = at::empty({O, I}, x.options());
    if (need_W) dW = at::empty({O, I, R}, x.options());
    const Tensor ga = grad_a.to(x.scalar_type()).contiguous(), xc = x.contiguous(), sc = contig_or_absent(s),
                 gc = grid.contiguous(), bw = contig_or_absent(base_weight), Wc = W.contiguous();
    const int code = dtype_code(x), mode = g_mode.load();
    Scratch* ws = scratch(x.device(), st, WS_EDGE_X,
                          kanb200_workspace_bytes(KANB200_OP_EDGE_X_BWD, mode, code, N, I, O, G, (int)k, 0, 0));
    {
        ScopedTimer timer("edge_backward", st);
        check_rc(kanb200_edge_abs_mean_x_backward(code, mode, ga.data_ptr(), xc.data_ptr(), cptr(sc), gc.data_ptr(), cptr(bw),
                                                  Wc.data_ptr(), mptr(gx), mptr(ds), mptr(dbw), mptr(dW), N, I, O, G,
                                                  (int)k, ws ? ws->buf.data_ptr() : nullptr,
                                                  ws ? (size_t)ws->buf.numel() : 0, st));
    }
    return std::make_tuple(gx, ds, dbw, dW);
}

// ------------------------------------------------------------------------------------------------
// dense differentiable formulas (any device): used while a backward pass is itself being recorded,
// so that higher-order derivatives are exact (kan_backward_composite, csrc/kan_cpu.cpp:301-345)
// ------------------------------------------------------------------------------------------------
Tensor safe_ratio(const Tensor& num, const Tensor& den) {
    const Tensor live = den.ne(0);
    return at::where(live, num / at::where(live, den, at::ones_like(den)), at::zeros_like(num));
}

// Cox-de Boor recurrence on the dense [B, I, T-1] indicator tensor; half-open spans, the last one
// closed, zero-length knot differences contribute zero.
Tensor dense_basis(const Tensor& x, const Tensor& grid, int64_t k) {
    const Tensor xq = x.unsqueeze(-1), t = grid.unsqueeze(0);
    const int64_t T = grid.size(1);
    const Tensor lo = t.slice(-1, 0, T - 1), hi = t.slice(-1, 1, T);
    const Tensor inside = xq.ge(lo).logical_and(xq.lt(hi));
    const Tensor closing = xq.ge(lo.slice(-1, T - 2, T - 1)).logical_and(xq.le(hi.slice(-1, T - 2, T - 1)));
    Tensor B = at::cat({inside.slice(-1, 0, T - 2), closing}, -1).to(x.scalar_type());
    for (int64_t d = 1; d <= k; ++d) {
        const int64_t m = B.size(-1) - 1;
        const Tensor left = safe_ratio(xq - t.slice(-1, 0, m), t.slice(-1, d, d + m) - t.slice(-1, 0, m));
        const Tensor right = safe_ratio(t.slice(-1, d + 1, d + 1 + m) - xq,
                                        t.slice(-1, d + 1, d + 1 + m) - t.slice(-1, 1, 1 + m));
        B = left * B.slice(-1, 0, m) + right * B.slice(-1, 1, m + 1);
    }
    return B;
}

Tensor dense_basis_derivative(const Tensor& x, const Tensor& grid, int64_t k) {
    const Tensor lower = dense_basis(x, grid, k - 1);
    const int64_t R = grid.size(1) - k - 1;
    const Tensor t = grid.unsqueeze(0);
    const Tensor l0 = lower.slice(-1, 0, R), l1 = lower.slice(-1, 1, R + 1);
    const Tensor a = safe_ratio(l0, (t.slice(-1, k, k + R) - t.slice(-1, 0, R)).expand_as(l0));
    const Tensor b = safe_ratio(l1, (t.slice(-1, k + 1, k + 1 + R) - t.slice(-1, 1, 1 + R)).expand_as(l1));
    return (a - b) * (double)k;
}

std::tuple<Tensor, Tensor, Tensor, Tensor> kan_backward_composite(const Tensor& D, const Tensor& x, const Tensor& grid,
                                                                  const Tensor& base_weight, const Tensor& spline_weight,
                                                                  const Tensor& spline_scaler, int64_t k,
                                                                  bool has_scaler) {
    const int64_t B = x.size(0), I = x.size(1), O = spline_weight.size(0), R = spline_weight.size(2);
    const Tensor H = dense_basis(x, grid, k);
    const Tensor W = has_scaler ? spline_weight * spline_scaler.unsqueeze(2) : spline_weight;
    const Tensor DtH = D.t().matmul(H.reshape({B, I * R})).reshape({O, I, R});
    Tensor g_spline, g_scaler, g_base;
    if (has_scaler) {
        g_spline = spline_scaler.unsqueeze(2) * DtH;
        g_scaler = (spline_weight * DtH).sum(2);
    } else {
        g_spline = DtH;
    }
    const Tensor dH = dense_basis_derivative(x, grid, k);
    Tensor gx = (D.matmul(W.reshape({O, I * R})).reshape({B, I, R}) * dH).sum(2);
    if (has(base_weight)) {
        g_base = D.t().matmul(at::silu(x));
        const Tensor sig = at::sigmoid(x);
        gx = gx + D.matmul(base_weight) * (sig * (1.0 + x * (1.0 - sig)));
    }
    return std::make_tuple(gx, g_base, g_spline, g_scaler);
}

// ------------------------------------------------------------------------------------------------
// gradient sinks: a data-parallel host may register, per layer (keyed by the storage of its
// spline_weight), a Python object that receives the parameter gradients directly -- the backward then
// writes them range by range of output rows into the sink's tensors (no autograd accumulation) and
// tells the sink after each range.  Protocol of the object: destinations(bw|None, sw, sc|None) ->
// (gb, gs, gc|None) | None;  row_ranges(O) -> [(o0, o1), ...];  rows_done(o0, o1).
// ------------------------------------------------------------------------------------------------
std::mutex g_sink_mutex;
std::unordered_map<uintptr_t, py::object> g_sinks;
std::atomic<int> g_sinks_disabled{0};

void register_grad_sink(const Tensor& spline_weight, py::object sink) {
    std::lock_guard<std::mutex> lock(g_sink_mutex);
    g_sinks[reinterpret_cast<uintptr_t>(spline_weight.data_ptr())] = std::move(sink);
}
void unregister_grad_sink(const Tensor& spline_weight) {
    std::lock_guard<std::mutex> lock(g_sink_mutex);
    g_sinks.erase(reinterpret_cast<uintptr_t>(spline_weight.data_ptr()));
}

struct NoGradSinks {
    void enter() { g_sinks_disabled.fetch_add(1); }
    bool exit(const py::object&, const py::object&, const py::object&) {
        g_sinks_disabled.fetch_sub(1);
        return false;
    }
};

// Returns true when the sink took the parameter gradients (then gx holds the input gradient if asked).
bool sink_backward(bool need_x, bool need_base, bool need_spline, bool need_scaler, const Tensor& grad_output,
                   const Tensor& x, const Tensor& grid, const Tensor& base_weight, const Tensor& spline_weight,
                   const Tensor& spline_scaler, int64_t k, bool has_scaler, Tensor& gx) {
    const bool has_base = has(base_weight);
    const bool wants_all = need_spline && (need_base || !has_base) && (need_scaler || !has_scaler);
    if (!wants_all || x.scalar_type() != at::kFloat || x.size(0) < 1) return false;
    const Dims d = check_inputs(x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler);
    const int mode = kanb200_resolve_mode(g_mode.load(), KANB200_F32, d.N, d.I, d.O, d.G, d.k);
    if (mode != KANB200_MODE_TC_BF16X3 && mode != KANB200_MODE_TC_BF16X1) return false;

    // The sink is a Python object: the interpreter lock is held for the rest of this function (the
    // thread that called backward() has released it while the engine runs; launches do not block).
    py::gil_scoped_acquire gil;
    Tensor gb, gs, gc;
    std::vector<std::pair<int64_t, int64_t>> ranges;
    py::object sink;
    {
        std::lock_guard<std::mutex> lock(g_sink_mutex);
        auto it = g_sinks.find(reinterpret_cast<uintptr_t>(spline_weight.data_ptr()));
        if (it == g_sinks.end()) return false;
        sink = it->second;
    }
    {
        py::object dest = sink.attr("destinations")(has_base ? py::cast(base_weight) : py::none(),
                                                    py::cast(spline_weight),
                                                    has_scaler ? py::cast(spline_scaler) : py::none());
        if (dest.is_none()) return false;
        py::tuple t = dest.cast<py::tuple>();
        gb = t[0].cast<Tensor>();
        gs = t[1].cast<Tensor>();
        if (!t[2].is_none()) gc = t[2].cast<Tensor>();
        for (auto item : sink.attr("row_ranges")(d.O)) {
            py::tuple r = item.cast<py::tuple>();
            ranges.emplace_back(r[0].cast<int64_t>(), r[1].cast<int64_t>());
        }
    }
    TORCH_CHECK(gb.is_contiguous() && gs.is_contiguous() && (!gc.defined() || gc.is_contiguous()),
                "gradient sink: destinations must be contiguous");
    c10::cuda::CUDAGuard guard(x.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const Tensor D = grad_output.to(x.scalar_type()).contiguous(), xc = x.contiguous(), gcn = grid.contiguous(),
                 bw = contig_or_absent(base_weight), sw = spline_weight.contiguous(),
                 sc = has_scaler ? contig_or_absent(spline_scaler) : Tensor();
    for (auto& r : ranges) {
        const size_t bytes = kanb200_workspace_bytes(KANB200_OP_BACKWARD, mode, KANB200_F32, d.N, d.I,
                                                     r.second - r.first, d.G, d.k, 0, 1);
        Scratch* ws = scratch(x.device(), st, WS_BWD, bytes);
        {
            ScopedTimer timer("backward", st);
            check_rc(kanb200_backward_param_rows(mode, D.data_ptr(), xc.data_ptr(), gcn.data_ptr(), cptr(bw),
                                                 sw.data_ptr(), cptr(sc), mptr(gb), gs.data_ptr(), mptr(gc), d.N, d.I,
                                                 d.O, d.G, d.k, r.first, r.second, ws->buf.data_ptr(),
                                                 (size_t)ws->buf.numel(), st));
        }
        sink.attr("rows_done")(r.first, r.second);
    }
    if (need_x)
        gx = backward_impl(grad_output, x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler, true, false,
                           false).gx;
    return true;
}

// ------------------------------------------------------------------------------------------------
// autograd node of the native layer (KANFunction, csrc/kan_autograd.cpp:13-111).  Saves the inputs
// only (no basis).  Backward: composite differentiable formulas while grad mode is on
// (create_graph=True), native kernels with un-needed gradients skipped otherwise.
// ------------------------------------------------------------------------------------------------
struct KANFunction : public torch::autograd::Function<KANFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& x, const Tensor& grid,
                          const Tensor& base_weight, const Tensor& spline_weight, const Tensor& spline_scaler,
                          int64_t spline_order, bool has_scaler) {
        ctx->saved_data["order"] = spline_order;
        ctx->saved_data["has_scaler"] = has_scaler;
        ctx->saved_data["allow_sink"] = g_sinks_disabled.load() == 0;
        Tensor y = forward_impl(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler);
        ctx->save_for_backward({x, grid, base_weight, spline_weight, spline_scaler});
        return y;
    }

    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                   torch::autograd::variable_list grad_outputs) {
        const auto saved = ctx->get_saved_variables();
        const Tensor &x = saved[0], &grid = saved[1], &base_weight = saved[2], &spline_weight = saved[3],
                     &spline_scaler = saved[4];
        const int64_t k = ctx->saved_data["order"].toInt();
        const bool has_scaler = ctx->saved_data["has_scaler"].toBool();
        const bool allow_sink = ctx->saved_data["allow_sink"].toBool();
        const bool has_base = has(base_weight);
        const Tensor& D = grad_outputs[0];
        Tensor gx, gb, gs, gc;
        if (at::GradMode::is_enabled()) {
            std::tie(gx, gb, gs, gc) =
                kan_backward_composite(D, x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler);
        } else {
            const bool need_x = ctx->needs_input_grad(0);
            const bool need_base = ctx->needs_input_grad(2) && has_base;
            const bool need_spline = ctx->needs_input_grad(3) || (has_scaler && ctx->needs_input_grad(4));
            bool sunk = false;
            bool any_sink;
            {
                std::lock_guard<std::mutex> lock(g_sink_mutex);
                any_sink = !g_sinks.empty();
            }
            if (any_sink && allow_sink)
                sunk = sink_backward(need_x, ctx->needs_input_grad(2), ctx->needs_input_grad(3),
                                     ctx->needs_input_grad(4), D, x, grid, base_weight, spline_weight, spline_scaler, k,
                                     has_scaler, gx);
            if (sunk) return {gx, Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
            Grads g = backward_impl(D, x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler, need_x,
                                    need_base, need_spline);
            gx = g.gx; gb = g.gb; gs = g.gs; gc = g.gc;
        }
        return {gx, Tensor(), has_base ? gb : Tensor(), gs, has_scaler ? gc : Tensor(), Tensor(), Tensor()};
    }
};

Tensor kan_apply(const Tensor& x, const Tensor& grid, const Tensor& base_weight, const Tensor& spline_weight,
                 const Tensor& spline_scaler, int64_t spline_order, bool has_scaler) {
    return KANFunction::apply(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler);
}

// ------------------------------------------------------------------------------------------------
// raw operators with the reference's schemas (csrc/kan_ext.cpp:62-75)
// ------------------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor> kan_forward(const Tensor& x, const Tensor& grid, const Tensor& base_weight,
                                       const Tensor& spline_weight, const Tensor& spline_scaler, int64_t spline_order,
                                       bool has_scaler) {
    Tensor y = forward_impl(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler);
    return std::make_tuple(y, basis(x, grid, spline_order));
}

// `basis` is accepted for schema compatibility and ignored: what the kernels need is recomputed from x.
std::tuple<Tensor, Tensor, Tensor, Tensor> kan_backward(const Tensor& grad_output, const Tensor& x, const Tensor& grid,
                                                        const Tensor& base_weight, const Tensor& spline_weight,
                                                        const Tensor& spline_scaler, const Tensor& /*basis*/,
                                                        int64_t spline_order, bool has_scaler) {
    Grads g = backward_impl(grad_output, x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler,
                            true, true, true);
    return std::make_tuple(g.gx, g.gb, g.gs, g.gc);
}

std::tuple<Tensor, Tensor, Tensor, Tensor> kan_backward_op(const Tensor& grad_output, const Tensor& x,
                                                           const Tensor& grid, const Tensor& base_weight,
                                                           const Tensor& spline_weight, const Tensor& spline_scaler,
                                                           const Tensor& basis_, int64_t spline_order, bool has_scaler) {
    Tensor gx, gb, gs, gc;
    std::tie(gx, gb, gs, gc) = kan_backward(grad_output, x, grid, base_weight, spline_weight, spline_scaler, basis_,
                                            spline_order, has_scaler);
    const Tensor empty = at::empty({0}, x.options());
    return std::make_tuple(gx, gb.defined() ? gb : empty, gs, gc.defined() ? gc : empty);
}

std::tuple<Tensor, Tensor> kan_forward_meta(const Tensor& x, const Tensor& grid, const Tensor& /*base_weight*/,
                                            const Tensor& spline_weight, const Tensor& /*spline_scaler*/,
                                            int64_t spline_order, bool /*has_scaler*/) {
    const int64_t R = grid.size(1) - spline_order - 1;
    return std::make_tuple(at::empty({x.size(0), spline_weight.size(0)}, x.options()),
                           at::empty({x.size(0), x.size(1), R}, x.options()));
}

std::tuple<Tensor, Tensor, Tensor, Tensor> kan_backward_meta(const Tensor& /*grad_output*/, const Tensor& x,
                                                             const Tensor& /*grid*/, const Tensor& base_weight,
                                                             const Tensor& spline_weight, const Tensor& spline_scaler,
                                                             const Tensor& /*basis*/, int64_t /*spline_order*/,
                                                             bool has_scaler) {
    const Tensor empty = at::empty({0}, x.options());
    return std::make_tuple(at::empty_like(x), base_weight.numel() > 0 ? at::empty_like(base_weight) : empty,
                           at::empty_like(spline_weight), has_scaler ? at::empty_like(spline_scaler) : empty);
}

}  // namespace

TORCH_LIBRARY(spline_kan, m) {
    m.def("kan_forward(Tensor x, Tensor grid, Tensor base_weight, Tensor spline_weight, Tensor spline_scaler, "
          "int spline_order, bool has_scaler) -> (Tensor output, Tensor basis)");
    m.def("kan_backward(Tensor grad_output, Tensor x, Tensor grid, Tensor base_weight, Tensor spline_weight, "
          "Tensor spline_scaler, Tensor basis, int spline_order, bool has_scaler) -> (Tensor grad_x, "
          "Tensor grad_base_weight, Tensor grad_spline_weight, Tensor grad_spline_scaler)");
}

TORCH_LIBRARY_IMPL(spline_kan, CUDA, m) {
    m.impl("kan_forward", &kan_forward);
    m.impl("kan_backward", &kan_backward_op);
}

TORCH_LIBRARY_IMPL(spline_kan, Meta, m) {
    m.impl("kan_forward", &kan_forward_meta);
    m.impl("kan_backward", &kan_backward_meta);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200-native operator layer of the KANLinear path (counterpart of spline_kan._C)";
    m.attr("CUDA_MAX_DEG0_BASIS") = KANB200_MAX_DEG0_BASIS;
    m.attr("CUDA_MAX_IN_FEATURES") = KANB200_MAX_IN_FEATURES;
    m.attr("HAS_FUSED_KERNELS") = true;
    m.attr("TORCH_OPS_REGISTERED") = true;
    if (std::getenv("KAN_B200_BACKTRACE")) install_backtrace_handler();
    if (const char* env = std::getenv("KAN_B200_MODE")) {
        const int mode = mode_from_name(env);
        if (mode >= 0) g_mode.store(mode);
    }

    m.def("kan_forward", &kan_forward, py::arg("x"), py::arg("grid"), py::arg("base_weight"),
          py::arg("spline_weight"), py::arg("spline_scaler"), py::arg("spline_order"), py::arg("has_scaler"),
          "(output [B, O], basis [B, I, R])");
    m.def("kan_backward",
          [](const Tensor& go, const Tensor& x, const Tensor& grid, const Tensor& bw, const Tensor& sw, const Tensor& sc,
             const Tensor& basis_, int64_t order, bool has_scaler) {
              Tensor gx, gb, gs, gc;
              std::tie(gx, gb, gs, gc) = kan_backward(go, x, grid, bw, sw, sc, basis_, order, has_scaler);
              auto opt = [](const Tensor& t) -> py::object { return t.defined() ? py::cast(t) : py::none(); };
              return py::make_tuple(opt(gx), opt(gb), opt(gs), opt(gc));
          },
          py::arg("grad_output"), py::arg("x"), py::arg("grid"), py::arg("base_weight"), py::arg("spline_weight"),
          py::arg("spline_scaler"), py::arg("basis"), py::arg("spline_order"), py::arg("has_scaler"),
          "(grad_x, grad_base_weight|None, grad_spline_weight, grad_spline_scaler|None)");
    m.def("kan_apply", &kan_apply, py::arg("x"), py::arg("grid"), py::arg("base_weight"), py::arg("spline_weight"),
          py::arg("spline_scaler"), py::arg("spline_order"), py::arg("has_scaler"),
          "autograd-aware forward; the call KANLinear uses");
    m.def("kan_backward_composite",
          [](const Tensor& go, const Tensor& x, const Tensor& grid, const Tensor& bw, const Tensor& sw, const Tensor& sc,
             int64_t order, bool has_scaler) {
              Tensor gx, gb, gs, gc;
              std::tie(gx, gb, gs, gc) = kan_backward_composite(go, x, grid, bw, sw, sc, order, has_scaler);
              auto opt = [](const Tensor& t) -> py::object { return t.defined() ? py::cast(t) : py::none(); };
              return py::make_tuple(opt(gx), opt(gb), opt(gs), opt(gc));
          },
          "backward from differentiable dense formulas (any device)");
    m.def("basis", &basis, py::arg("x"), py::arg("grid"), py::arg("spline_order"), "dense basis H [B, I, R]");
    m.def("basis_grad", &basis_grad, py::arg("x"), py::arg("grid"), py::arg("spline_order"), py::arg("grad_basis"),
          "gx[b,i] = sum_r gH[b,i,r] dB_r/dx");
    m.def("edge_abs_mean", &edge_abs_mean, py::arg("s"), py::arg("H"), py::arg("base_weight"), py::arg("W"),
          "a[o,i] = mean_n |s bw + <H, W>| without phi [N,O,I]");
    m.def("edge_abs_mean_backward",
          [](const Tensor& ga, const Tensor& s, const Tensor& H, const Tensor& bw, const Tensor& W, bool need_s,
             bool need_H, bool need_bw, bool need_W) {
              Tensor ds, dH, dbw, dW;
              std::tie(ds, dH, dbw, dW) = edge_abs_mean_backward(ga, s, H, bw, W, need_s, need_H, need_bw, need_W);
              auto opt = [](const Tensor& t) -> py::object { return t.defined() ? py::cast(t) : py::none(); };
              return py::make_tuple(opt(ds), opt(dH), opt(dbw), opt(dW));
          },
          py::arg("grad_a"), py::arg("s"), py::arg("H"), py::arg("base_weight"), py::arg("W"), py::arg("need_s"),
          py::arg("need_H"), py::arg("need_bw"), py::arg("need_W"), "(ds|None, dH|None, dbw|None, dW|None)");
    m.def("edge_abs_mean_x", &edge_abs_mean_x, py::arg("x"), py::arg("s"), py::arg("grid"), py::arg("base_weight"),
          py::arg("W"), py::arg("spline_order"),
          "a[o,i] = mean_n |s bw + <B(x), W>| straight from x; s empty = silu(x)");
    m.def("prepare_forward", &prepare_forward, py::arg("grid"), py::arg("base_weight"), py::arg("spline_weight"),
          py::arg("spline_scaler"), py::arg("spline_order"), py::arg("has_scaler"),
          "table + weight image of a layer with fixed parameters (empty = no prepared form)");
    m.def("forward_prepared", &forward_prepared, py::arg("x"), py::arg("prepared"), py::arg("out_features"),
          py::arg("grid_size"), py::arg("spline_order"), py::arg("has_base"),
          "layer(x) from x and the buffer of prepare_forward: the contraction alone");
    m.def("resolve_mode",
          [](int64_t N, int64_t I, int64_t O, int64_t G, int64_t k, bool f64) {
              return kanb200_resolve_mode_for(KANB200_OP_FORWARD, g_mode.load(), f64 ? KANB200_F64 : KANB200_F32, N, I, O,
                                              (int)G, (int)k);
          },
          "the kernel family (KANB200_MODE_*) a forward call of this shape takes in the current mode");
    m.def("edge_penalty", &edge_penalty, py::arg("a"), py::arg("mu1"), py::arg("mu2"),
          "(mu1 sum(a) + mu2 entropy(a / sum(a)), its gradient with respect to a) in one launch");
    m.def("edge_abs_mean_x_backward",
          [](const Tensor& ga, const Tensor& x, const Tensor& s, const Tensor& grid, const Tensor& bw, const Tensor& W,
             int64_t k, bool need_x, bool need_s, bool need_bw, bool need_W) {
              Tensor gx, ds, dbw, dW;
              std::tie(gx, ds, dbw, dW) = edge_abs_mean_x_backward(ga, x, s, grid, bw, W, k, need_x, need_s, need_bw, need_W);
              auto opt = [](const Tensor& t) -> py::object { return t.defined() ? py::cast(t) : py::none(); };
              return py::make_tuple(opt(gx), opt(ds), opt(dbw), opt(dW));
          },
          py::arg("grad_a"), py::arg("x"), py::arg("s"), py::arg("grid"), py::arg("base_weight"), py::arg("W"),
          py::arg("spline_order"), py::arg("need_x"), py::arg("need_s"), py::arg("need_bw"), py::arg("need_W"),
          "(gx|None, ds|None, dbw|None, dW|None)");
    m.def("set_basis_impl", [](int impl) { check_rc(kanb200_set_basis_impl(impl)); }, py::arg("impl"));
    m.def("get_basis_impl", []() { return kanb200_get_basis_impl(); });

    m.def("set_mma_mode",
          [](const std::string& name) {
              const int mode = mode_from_name(name);
              if (mode < 0) throw py::value_error("mode must be one of ['auto', 'bf16x1', 'bf16x3', 'simt'], got '" + name + "'");
              g_mode.store(mode);
          },
          "arithmetic of the fp32 contraction: auto, simt, bf16x3 (split operands, fp32-level accuracy) or bf16x1");
    m.def("get_mma_mode", []() { return std::string(mode_name(g_mode.load())); });
    m.def("register_grad_sink", &register_grad_sink);
    m.def("unregister_grad_sink", &unregister_grad_sink);
    py::class_<NoGradSinks>(m, "no_grad_sinks",
                            "context in which forwards do not use a registered gradient sink: for call sites whose "
                            "parameters also receive gradients from other terms")
        .def(py::init<>())
        .def("__enter__", &NoGradSinks::enter)
        .def("__exit__", &NoGradSinks::exit);
    m.def("check_status", &check_status_all,
          "synchronises and raises if a tensor-core kernel reported a timed-out wait on any scratch buffer");
    m.def("release_workspaces", &release_workspaces);
    m.def("_poke_status", &poke_status, py::arg("purpose"), py::arg("code"), py::arg("as_kernel") = true);
    m.def("set_event_log", &set_event_log);
    m.def("take_event_log", &take_event_log);
}
