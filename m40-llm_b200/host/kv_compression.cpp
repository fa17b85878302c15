#include "kv_compression.hpp"

namespace m40host {

const char* to_string(KvExactOldBacking b) {
    switch (b) {
        case KvExactOldBacking::Dense: return "dense";
        case KvExactOldBacking::Q8: return "q8";
        default: return "fp16-k-q4-v";
    }
}

const char* to_string(KvExactOldAttention a) {
    switch (a) {
        case KvExactOldAttention::Staged: return "staged";
        case KvExactOldAttention::Q8Direct: return "q8-direct";
        default: return "fp16-k-q4-v-direct";
    }
}

KvCompressionConfig KvCompressionConfig::dense_reference() {
    KvCompressionConfig c;
    c.mode = KvCompressMode::Off;
    c.exact_old_backing = KvExactOldBacking::Dense;
    c.exact_old_attention = KvExactOldAttention::Staged;
    return c;
}

KvCompressionConfig KvCompressionConfig::for_mode(KvCompressMode mode) {
    KvCompressionConfig c = mode == KvCompressMode::BlockSelectExact ? KvCompressionConfig() : dense_reference();
    c.mode = mode;
    return c;
}

std::string KvCompressionConfig::validate() const {
    if (recent_window == 0) return "kv_recent_window must be > 0";
    if (block_size == 0) return "kv_compress_block must be > 0";
    const bool select = mode == KvCompressMode::BlockSelectExact || mode == KvCompressMode::BlockSelectLossy;
    if (select && top_blocks == 0) return "kv_compress_top_blocks must be > 0 for block-select modes";
    if (exact_old_backing != KvExactOldBacking::Dense && mode != KvCompressMode::BlockSelectExact)
        return std::string("kv_exact_old_backing=") + to_string(exact_old_backing) +
               " requires kv_compress_mode=block-select-exact";
    switch (exact_old_attention) {
        case KvExactOldAttention::Staged: break;
        case KvExactOldAttention::Q8Direct:
            if (exact_old_backing != KvExactOldBacking::Q8)
                return "kv_exact_old_attention=q8-direct requires kv_exact_old_backing=q8";
            break;
        case KvExactOldAttention::Fp16KQ4VDirect:
            if (exact_old_backing != KvExactOldBacking::Fp16KQ4V)
                return "kv_exact_old_attention=fp16-k-q4-v-direct requires kv_exact_old_backing=fp16-k-q4-v";
            break;
    }
    return "";
}

std::string KvCompressionConfig::validate_runtime_support(uint32_t max_seq_len, uint32_t head_dim) const {
    std::string e = validate();
    if (!e.empty()) return e;
    if (mode == KvCompressMode::Off) return "";
    if (max_seq_len == 0) return "compressed KV requires model context_length > 0";
    if (recent_window > max_seq_len)
        return "kv_recent_window " + std::to_string(recent_window) + " exceeds model context_length " +
               std::to_string(max_seq_len) + "; use a smaller --kv-recent-window or --kv-compress-mode off";
    if (block_size > max_seq_len)
        return "kv_compress_block " + std::to_string(block_size) + " exceeds model context_length " +
               std::to_string(max_seq_len);
    const bool select = mode == KvCompressMode::BlockSelectExact || mode == KvCompressMode::BlockSelectLossy;
    if (select && top_blocks > 64)
        return "kv_compress_top_blocks " + std::to_string(top_blocks) + " exceeds the CUDA block-select limit of 64";
    if (mode != KvCompressMode::BlockSelectExact) {
        if (head_dim != 64) return "mode currently requires head_dim=64, got head_dim=" + std::to_string(head_dim);
        return "";
    }
    if (head_dim == 64) return "";
    if (head_dim == 128 && exact_old_backing == KvExactOldBacking::Fp16KQ4V &&
        exact_old_attention == KvExactOldAttention::Fp16KQ4VDirect)
        return "";
    return std::string("block-select-exact currently requires head_dim=64, or head_dim=128 with "
                       "--kv-exact-old-backing fp16-k-q4-v and --kv-exact-old-attention fp16-k-q4-v-direct; got head_dim=") +
           std::to_string(head_dim) + " backing=" + to_string(exact_old_backing) +
           " attention=" + to_string(exact_old_attention);
}

std::string KvCompressionConfig::validate_b200_support(uint32_t max_seq_len, uint32_t head_dim) const {
    std::string e = validate_runtime_support(max_seq_len, head_dim);
    if (!e.empty()) return e;
    if (mode == KvCompressMode::Off) return "";
    if (mode == KvCompressMode::BlockSelectExact && exact_old_backing == KvExactOldBacking::Fp16KQ4V &&
        exact_old_attention == KvExactOldAttention::Fp16KQ4VDirect)
        return "";
    return "this build implements kv_compress_mode=off and block-select-exact with fp16-k-q4-v / fp16-k-q4-v-direct only";
}

}  // namespace m40host
