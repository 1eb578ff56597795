// attn_decode_static_scratch(): decode attention for callers that must not allocate.
//
// Some hosts of this library cannot give attn_decode() a workspace: a serving loop that handed
// every free byte of HBM to its KV-cache pool at start-up (a later cudaMalloc may fail, and it
// stalls the device while it runs), or code embedded where only the host application's own
// allocator may touch the device heap. For them the split-KV partials live in a fixed array that
// is part of this library's device image, so no allocation call is ever made on their behalf.
//
// Cost and limits:
//   * the array is ATTN_STATIC_SCRATCH_BYTES (8 MiB) and is held, until the process exits, on every
//     GPU on which this library is loaded;
//   * shapes whose partials need more than that are refused with ATTN_ERR_WORKSPACE (for 32/8 heads
//     of dim 128 that is a batch above ~340 sequences);
//   * all calls on one GPU share the one array: two calls that overlap in time on the GPU (different
//     streams) overwrite each other's partials. Serialise them on one stream, or give the
//     overlapping call its own workspace through attn_decode();
//   * the array keeps whatever the previous call left in it. That is harmless here: the split
//     pass writes every partial before the merge pass reads it, and the arrival counters that would
//     have to start at zero belong to the single-launch kernel, which this entry point does not use;
//   * the first call on a device looks up the array's device address (one cudaGetSymbolAddress with
//     that device current, checked, cached). Under CUDA's default lazy module loading this lookup
//     is also the moment the module that holds the array is loaded and its 8 MiB are reserved, so
//     the first call belongs at start-up: before the host gives the rest of the HBM away (later it
//     could fail with out-of-memory, reported as ATTN_ERR_CUDA) and outside any stream capture.
//     CUDA_MODULE_LOADING=EAGER moves the reservation to the time the library is loaded.
#include "attn_internal.cuh"

namespace {

// The name below is a host-side handle in host code, not a device address: the address that
// kernels can use is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[ATTN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_ptr[kMaxDevices];

int static_scratch_address(void** out) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ATTN_ERR_DEVICE;
    void* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return ATTN_ERR_CUDA;
        g_scratch_ptr[dev].store(p, std::memory_order_release);  // same value from every thread
    }
    *out = p;
    return ATTN_OK;
}

}  // namespace

extern "C" int attn_decode_static_scratch(const AttnDecodeArgs* args, void* stream) {
    if (!args) return ATTN_ERR_INVALID_ARG;
    const size_t need = attn_decode_workspace_bytes(args->batch, args->n_heads, args->n_kv_heads, args->head_dim);
    if (need == 0) return ATTN_ERR_UNSUPPORTED;
    if (need > static_cast<size_t>(ATTN_STATIC_SCRATCH_BYTES)) return ATTN_ERR_WORKSPACE;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != ATTN_OK) return rc;
    AttnDecodeArgs a = *args;  // the caller's inputs and outputs, our scratch
    a.workspace = scratch;
    a.workspace_bytes = ATTN_STATIC_SCRATCH_BYTES;
    return attn_decode(&a, stream);
}
