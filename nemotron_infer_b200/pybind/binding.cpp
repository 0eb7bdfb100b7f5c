// pybind11 module with the reference's Python-visible surface for the hot-path ops.
//
// The reference exposes one pybind11 module, `binding` (binding.cu:210-246), whose functions take device
// addresses as integers.  This module keeps, for the ops this library implements, the same names, argument
// order and None return (embedding, rmsnorm, sync, reset_allocator, free_allocator and the model constants),
// and adds the fused / block-internal ops under new names.  It is a thin veneer over the C ABI in
// include/nemotron_b200.h; a call the library rejects raises RuntimeError instead of being undefined behaviour.
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "nemotron_b200.h"

namespace py = pybind11;

namespace cfg {   // binding.cu:35-46
constexpr int HIDDEN = 3136;
constexpr int H = 96, P = 80, N = 128, G = 8, CONV_K = 4;
constexpr int H_Q = 40, H_KV = 8, HEAD = 128;
constexpr int INTER = 12544;
constexpr int VOCAB = 131072;
constexpr float EPS = 1e-5f;
}  // namespace cfg

static inline const void* cp(uintptr_t p) { return reinterpret_cast<const void*>(p); }
static inline void* mp(uintptr_t p) { return reinterpret_cast<void*>(p); }
static inline const float* fp(uintptr_t p) { return reinterpret_cast<const float*>(p); }

static void check(int status, const char* what) {
    if (status == NMT_OK) return;
    std::string msg = std::string(what) + ": " + nmt_status_string(status);
    if (status == NMT_ERR_LAUNCH) msg += std::string(" (") + nmt_last_cuda_error() + ")";
    throw std::runtime_error(msg);
}

static void* g_stream = nullptr;   // legacy default stream, as at every reference call site (binding.cu:72)

PYBIND11_MODULE(binding, m) {
    m.doc() = "nemotron_infer hot-path ops on libnemotron_b200 (B200, sm_100a)";
    m.attr("HIDDEN") = cfg::HIDDEN;
    m.attr("H") = cfg::H;
    m.attr("P") = cfg::P;
    m.attr("N") = cfg::N;
    m.attr("G") = cfg::G;
    m.attr("CONV_K") = cfg::CONV_K;
    m.attr("H_Q") = cfg::H_Q;
    m.attr("H_KV") = cfg::H_KV;
    m.attr("HEAD") = cfg::HEAD;
    m.attr("INTER") = cfg::INTER;
    m.attr("VOCAB") = cfg::VOCAB;
    m.attr("CONV_DIM") = cfg::H * cfg::P + 2 * cfg::G * cfg::N;
    m.attr("IN_PROJ") = cfg::H * cfg::P + (cfg::H * cfg::P + 2 * cfg::G * cfg::N) + cfg::H;

    // --- names the reference has (binding.cu:228-232) ---
    m.def("reset_allocator", [] {});   // these kernels use no workspace
    m.def("free_allocator", [] {});
    m.def("sync", [] { check(nmt_device_synchronize(), "sync"); });
    m.def("embedding", [](uintptr_t table, uintptr_t ids, uintptr_t out, int num_tokens) {
        check(nmt_embedding_bf16_i64(cp(table), reinterpret_cast<const int64_t*>(ids), mp(out), num_tokens, cfg::HIDDEN, 0,
                                     nullptr, g_stream), "embedding");
    });
    m.def("rmsnorm", [](uintptr_t in, uintptr_t out, uintptr_t w, int M) {
        check(nmt_rmsnorm_bf16(cp(in), mp(out), fp(w), M, cfg::HIDDEN, cfg::EPS, g_stream), "rmsnorm");
    });

    // --- additions ---
    m.def("set_stream", [](uintptr_t stream) { g_stream = reinterpret_cast<void*>(stream); },
          "cudaStream_t (as an int) later calls enqueue on; 0 = legacy default stream");
    m.def("set_device", [](int device) { check(nmt_set_device(device), "set_device"); });
    m.def("add_rmsnorm", [](uintptr_t x, uintptr_t r, uintptr_t w, uintptr_t out_res, uintptr_t out, int M) {
        check(nmt_add_rmsnorm_bf16(cp(x), cp(r), fp(w), mp(out_res), mp(out), M, cfg::HIDDEN, cfg::EPS, g_stream), "add_rmsnorm");
    }, "out_res = x + r; out = rmsnorm(out_res) * w   (block-tail add fused with the next block's pre-norm)");
    m.def("rmsnorm_gated", [](uintptr_t y, uintptr_t z, uintptr_t w, uintptr_t out, int M) {
        check(nmt_rmsnorm_gated_bf16(cp(y), cp(z), fp(w), mp(out), M, cfg::H * cfg::P, cfg::H * cfg::P / cfg::G, cfg::EPS,
                                     g_stream), "rmsnorm_gated");
    }, "Mamba-2 gated RMSNorm at the model's shape (7680 channels, 8 groups)");
    m.def("relu2", [](uintptr_t u, uintptr_t out, int M) {
        check(nmt_relu2_bf16(cp(u), mp(out), static_cast<int64_t>(M) * cfg::INTER, g_stream), "relu2");
    });
    m.def("add", [](uintptr_t a, uintptr_t b, uintptr_t out, int M) {
        check(nmt_add_bf16(cp(a), cp(b), mp(out), static_cast<int64_t>(M) * cfg::HIDDEN, g_stream), "add");
    });
    m.def("quantize_fp8", [](uintptr_t x, uintptr_t out, uintptr_t scale, uintptr_t amax, int64_t n) {
        check(nmt_quantize_fp8(cp(x), mp(out), reinterpret_cast<float*>(scale), reinterpret_cast<unsigned int*>(amax), n,
                               g_stream), "quantize_fp8");
    });
    m.def("fuse_next_norm", [](uintptr_t next_norm_w) { check(nmt_fuse_next_norm(fp(next_norm_w), cfg::EPS), "fuse_next_norm"); },
          "announce block i+1's norm weight (0 withdraws) before calling block i: the reference's blocks built on the "
          "drop-in headers then fuse block i's residual add with block i+1's pre-norm");
    m.def("fusion_reset", [] { check(nmt_fusion_reset(), "fusion_reset"); });
    m.def("fusion_counters", [] {
        int64_t fused = 0, skipped = 0;
        check(nmt_fusion_counters(&fused, &skipped), "fusion_counters");
        return py::make_tuple(fused, skipped);
    });
    m.def("version", [] { return std::string(nmt_version()); });
}
