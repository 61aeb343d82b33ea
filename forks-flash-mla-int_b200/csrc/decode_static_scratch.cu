// Split-KV sparse-MLA decode for hosts that must not allocate device memory at call time.
//
// Some callers of this library cannot call cudaMalloc (nor let a library do it for them): a serving
// engine that has handed every free byte of HBM to its own KV-cache pool at start-up has nothing left
// for a driver allocation in the middle of a decode step; cudaMalloc also synchronises the whole
// device, which a latency-bound decode loop cannot afford, and is not permitted while a stream is
// being captured.  The regular entry point, smla_sparse_mla_decode, leaves the split-KV scratch to the
// caller (the torch binding takes it from torch's caching allocator).  This variant brings its own:
// a fixed array that is part of the library image, so every GPU that loads the library holds
// kStaticScratchBytes of it until the process exits.
//
// The array's name is only a host-side handle.  Its device address is looked up once per device with
// cudaGetSymbolAddress, with that device current, on the first call made on that device -- make that
// first call outside any stream capture.  All calls on a device share the one array and it keeps
// whatever the previous call left in it; nothing in it has to start at zero (every partial the
// combine kernel reads is written by the attention kernel of the same call), but two calls whose
// kernels overlap on the GPU (different streams, or graphs replayed concurrently) race on it.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "smla_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = SMLA_STATIC_SCRATCH_BYTES;   // 64 MiB: two partial slots per CTA of a 148-SM part need 39 MB

static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_addr[64] = {};
bool g_scratch_ready[64] = {};

// Device address of the array on the CURRENT device (looked up once per device).
int static_scratch_address(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= 64) return SMLA_ETOOBIG;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ready[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (ptr == nullptr) return SMLA_EINVAL;
        g_scratch_addr[dev] = ptr;
        g_scratch_ready[dev] = true;
    }
    *out = g_scratch_addr[dev];
    return SMLA_OK;
}

}  // namespace

extern "C" {

int smla_sparse_mla_decode_static_scratch(const smla_attn_params_t *p, void *stream) {
    if (!p) return SMLA_EINVAL;
    if (p->num_splits < 0) return SMLA_EINVAL;
    int splits = p->num_splits;
    if (splits == 0) {   // same policy as smla_sparse_mla_decode (also checks the architecture)
        const int width = p->swa.topk + (p->extra.cache ? p->extra.topk : 0);
        const int rc = smla_decode_plan(p->num_tokens, p->num_heads, width, &splits, nullptr);
        if (rc != SMLA_OK) return rc;
    } else {
        int unused = 0;
        const int rc = smla_decode_plan(1, 1, 1, &unused, nullptr);   // architecture check only
        if (rc != SMLA_OK) return rc;
    }
    void *scratch = nullptr;
    if (splits > 1) {
        const long long want = static_cast<long long>(smla_attn_workspace_bytes(p->num_tokens, p->num_heads, splits));
        if (p->num_splits > 1) {
            // An explicit request is taken at its word, as by smla_sparse_mla_decode: it must fit as asked.
            if (want > static_cast<long long>(kStaticScratchBytes)) return SMLA_ETOOBIG;
        } else {
            // The automatic choice only sizes scratch, and what the kernels touch does not grow with the
            // token count: two partial slots of one head block per CTA plus 64 bytes per SM (39 MB on a
            // 148-SM part at 64 heads per block), whatever smla_attn_workspace_bytes says for many tokens.
            // The array is offered whole, the launcher takes as many CTAs as fit into it; the unsplit
            // schedule is used only when not even two fit.
            int dev = 0, sms = 0;
            cudaError_t e = cudaGetDevice(&dev);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return static_cast<int>(e);
            const long long have = std::min<long long>(want, static_cast<long long>(kStaticScratchBytes));
            if (smla::balanced_ctas(sms, smla::head_pad(p->num_heads), have) < 2) splits = 1;
        }
    }
    if (splits > 1) {
        const int rc = static_scratch_address(&scratch);
        if (rc != SMLA_OK) return rc;
    }
    return smla::launch_sparse_mla_attention(*p, splits, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
