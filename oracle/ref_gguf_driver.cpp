// Test infrastructure only. C-ABI driver around the reference's own GGUF parser (src/gguf.cpp, compiled from where it
// lies, include/gguf.hpp unmodified): opens a file the way the engine does (GGUF::GGUF, parse_llama_config,
// get_tensor) and reports what it found, so that files written by this repository's writer can be checked against
// the reader they are meant for.
#include <gguf.hpp>

#include <cstdint>
#include <cstring>
#include <string>

extern "C" {

struct RefGgufSummary {
    uint64_t tensor_count, context_length, embedding_length, block_count, feed_forward_length, rope_dimension_count,
        attention_head_count, attention_head_count_kv, vocab_size;
    float rope_freq_base, layer_norm_rms_epsilon;
    uint32_t alignment, quantization_version;
    char architecture[32];
    char error[256];
};

// 0 on success; -1 with `error` filled when the parser throws or the llama configuration is incomplete.
int ref_gguf_open(const char* path, RefGgufSummary* out) {
    std::memset(out, 0, sizeof(*out));
    try {
        GGUF g{std::filesystem::path(path)};
        out->tensor_count = g.tensor_count();
        out->alignment = g.alignment();
        out->quantization_version = g.quantization_version();
        std::strncpy(out->architecture, g.architecture().c_str(), sizeof(out->architecture) - 1);
        auto cfg = g.parse_llama_config();
        if (!cfg) {
            std::strncpy(out->error, "parse_llama_config returned nothing", sizeof(out->error) - 1);
            return -1;
        }
        out->context_length = cfg->context_length;
        out->embedding_length = cfg->embedding_length;
        out->block_count = cfg->block_count;
        out->feed_forward_length = cfg->feed_forward_length;
        out->rope_dimension_count = cfg->rope_dimension_count;
        out->attention_head_count = cfg->attention_head_count;
        out->attention_head_count_kv = cfg->kv_head_count();
        out->vocab_size = cfg->vocab_size;
        out->rope_freq_base = cfg->rope_freq_base;
        out->layer_norm_rms_epsilon = cfg->layer_norm_rms_epsilon;
        return 0;
    } catch (const std::exception& e) {
        std::strncpy(out->error, e.what(), sizeof(out->error) - 1);
        return -1;
    }
}

// Looks a tensor up by name: fills dims (up to 4, fastest first), the GGML type and the first `n_bytes` bytes of its
// data. Returns the number of dimensions, or -1 when the tensor is missing or the file does not parse.
int ref_gguf_tensor(const char* path, const char* name, uint64_t* dims, uint32_t* type, uint8_t* bytes, uint64_t n_bytes) {
    try {
        GGUF g{std::filesystem::path(path)};
        const TensorInfo* t = g.get_tensor(name);
        if (!t || t->n_dimensions > 4) return -1;
        for (uint32_t i = 0; i < t->n_dimensions; ++i) dims[i] = t->dimensions[i];
        *type = static_cast<uint32_t>(t->type);
        if (bytes && n_bytes) std::memcpy(bytes, t->data, n_bytes);
        return static_cast<int>(t->n_dimensions);
    } catch (const std::exception&) {
        return -1;
    }
}

}  // extern "C"
