// Library identity, status text, device selection and the tuning-knob table.
#include <cstring>
#include <cstdio>

#include "nmt_common.cuh"

namespace nmt {

std::atomic<int64_t> g_launches{0};
static thread_local char t_cuda_err[256] = "";
static thread_local int64_t t_launch_epoch = 0;
int64_t thread_launch_epoch() { return t_launch_epoch; }

int finish_launch(int n_kernels) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
        return NMT_ERR_LAUNCH;
    }
    g_launches.fetch_add(n_kernels, std::memory_order_relaxed);
    if (n_kernels > 0) ++t_launch_epoch;
    return NMT_OK;
}

// Knobs are plain ints read at launch time.  0 means "let the launcher decide".
struct Knob { const char* key; std::atomic<int> value; };
static Knob g_knobs[] = {
    {"ssm.rows_per_warp", {0}},   // SSM decode step: rows of a head a warp handles together (1, 2, 4 or 5; default: by rows per head)
    {"launch.pdl", {0}},          // 1 = launch with programmatic stream serialization (default), 2 = plain launches
    // add_rmsnorm / rmsnorm (bf16)
    {"norm.cluster", {0}},        // RMSNorm: 0 = cluster of CTAs per row only for rows one CTA cannot hold, 2/4/8 = always, 1 = never
    {"norm.cluster_staged", {0}}, // cluster RMSNorm: 1 (default) = row shares staged in shared memory by bulk copies, 2 = registers only
    {"norm.cluster_stages", {0}}, // cluster RMSNorm (staged): ring depth, 2..4 (default: what fits 200 KB)
    {"norm.staged_single", {0}},  // plain RMSNorm, 20,480 - 32,768 columns: 1 (default) = row staged in shared memory, 2 = register kernel
    {"norm.cluster_block", {0}},  // cluster RMSNorm: threads per CTA, 512 (default) or 256
    {"norm.cluster_ctas_per_sm", {0}},  // cluster RMSNorm: CTAs per SM the grid is sized for (default 3)
    {"norm.block", {0}},          // threads per CTA (= per row); 0 = by width
    {"norm.ctas_per_sm", {0}},    // >0: persistent grid of 148*k CTAs; 0: one pass, grid = rows/warps
    {"norm.rows_per_cta", {0}},   // CTA-per-row variant: rows a CTA loads together (1 or 2)
    {"quant.rows_per_cta", {0}},  // rows a CTA of the norm -> e4m3 pass handles together (1, 2 or 4)
    {"conv.chunk", {0}},          // causal conv1d: time steps per thread (4, 8, 16, 32 or 64)
    {"conv.pairs", {0}},          // causal conv1d: channel pairs per thread (2 = 8-byte vectors, 4 = 16-byte vectors)
    {"conv.unroll", {0}},         // causal conv1d: loads issued ahead of use (4 or 8)
    {"gemv.split", {0}},          // W8A16 GEMV: K-slices per row (1, 2, 4, 8); 0 = by K
    {"gemv.variant", {0}},        // W8A16 GEMV: 5 = tcgen05.mma fed by TMA (x as two e4m3 terms), 3 = mma.sync inner product, 1 = whole-unit CUDA-core loads, 2 = looped loads
    {"gemv.ring_stages", {0}},    // W8A16 GEMV (variant 5): 16 KB stages of the weight ring per CTA (default 4)
    {"gemv.kparts", {0}},         // W8A16 GEMV (variant 5): CTAs per row tile that split K = cluster size, 1 / 2 / 4 / 8; 0 = by shape
    {"gemv.early_trigger", {0}},  // W8A16 GEMV (mma): 1 (default) = let the next kernel launch once this one's last loads are issued, 2 = at the very end
    {"gemv.unit_chunks", {0}},    // W8A16 GEMV (mma): largest number of 64-k chunks per work unit (default 7)
    {"gemv.streams", {0}},        // W8A16 GEMV (mma): k-streams per 16-row tile (1, 2, 4, 8); 0 = by shape
    {"gemv.ctas_per_sm", {0}},    // W8A16 GEMV: persistent CTAs per SM; 0 = by shared-memory footprint
    // gated rmsnorm (bf16)
    {"gated.block", {0}},
    {"gated.ctas_per_sm", {0}},
    {"gated.rows_per_iter", {0}},
    // relu2 / add (bf16)
    {"ew.block", {0}},
    {"ew.unroll", {0}},
    {"ew.ctas_per_sm", {0}},
    // embedding gather
    {"emb.variant", {0}},         // 0 = by batch size, 1 = warp-per-row registers, 2 = TMA row relay
    {"emb.block", {0}},
    {"emb.ctas_per_sm", {0}},
    {"emb.relay_warps", {0}},     // relays (warps) per CTA of the TMA variant
    {"emb.tma_stages", {0}},
};
static Knob* find_knob(const char* key) {
    if (!key) return nullptr;
    for (auto& k : g_knobs) if (std::strcmp(k.key, key) == 0) return &k;
    return nullptr;
}
// Each TMA translation unit keeps its own device counter of timed-out waits and registers a reader here.
static cudaError_t (*g_timeout_readers[16])(unsigned int*);
static int g_n_timeout_readers = 0;
void register_timeout_reader(cudaError_t (*reader)(unsigned int*)) {
    if (g_n_timeout_readers < 16) g_timeout_readers[g_n_timeout_readers++] = reader;
}
int64_t read_wait_timeouts() {
    int64_t total = 0;
    for (int i = 0; i < g_n_timeout_readers; ++i) {
        unsigned int v = 0;
        if (g_timeout_readers[i](&v) != cudaSuccess) return -1;
        total += v;
    }
    return total;
}

bool pdl_enabled() {
    static Knob* const k = find_knob("launch.pdl");
    return k->value.load(std::memory_order_relaxed) != 2;
}

int tune(const char* key, int dflt) {
    Knob* k = find_knob(key);
    if (!k) return dflt;
    int v = k->value.load(std::memory_order_relaxed);
    return v > 0 ? v : dflt;
}

}  // namespace nmt

extern "C" {

const char* nmt_version(void) { return "nemotron_b200 0.1 (sm_100a)"; }

const char* nmt_status_string(int s) {
    switch (s) {
        case NMT_OK: return "ok";
        case NMT_ERR_NULL: return "null pointer";
        case NMT_ERR_ALIGN: return "pointer not aligned to the contract (16 bytes for bf16 tensors and for the fp32 weight / tap / bias vectors of the bf16 entry points, 4 bytes in the fp32 twins)";
        case NMT_ERR_SHAPE: return "bad shape (negative size, cols % 8 != 0, or group size does not divide cols)";
        case NMT_ERR_LAUNCH: return "CUDA launch failed (see nmt_last_cuda_error)";
        case NMT_ERR_UNSUPPORTED: return "unsupported shape or unknown tuning key";
        case NMT_ERR_TOO_LARGE: return "rows exceed NMT_STATIC_SCRATCH_MAX_ROWS, the capacity of the built-in scratch; use the workspace form";
        default: return "unknown status";
    }
}

const char* nmt_last_cuda_error(void) { return nmt::t_cuda_err; }

int nmt_set_device(int device) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        snprintf(nmt::t_cuda_err, sizeof(nmt::t_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
        return NMT_ERR_LAUNCH;
    }
    return NMT_OK;
}

int nmt_device_synchronize(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        snprintf(nmt::t_cuda_err, sizeof(nmt::t_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
        return NMT_ERR_LAUNCH;
    }
    return NMT_OK;
}

int nmt_tune_set(const char* key, int value) {
    nmt::Knob* k = nmt::find_knob(key);
    if (!k) return NMT_ERR_UNSUPPORTED;
    k->value.store(value, std::memory_order_relaxed);
    return NMT_OK;
}
int nmt_tune_get(const char* key, int* value) {
    nmt::Knob* k = nmt::find_knob(key);
    if (!k || !value) return NMT_ERR_UNSUPPORTED;
    *value = k->value.load(std::memory_order_relaxed);
    return NMT_OK;
}
int64_t nmt_device_wait_timeouts(void) { return nmt::read_wait_timeouts(); }
int64_t nmt_launch_count(void) { return nmt::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
