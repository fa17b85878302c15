// KV compression configuration of the decode path: the host-side mirror of the reference's
// src/kv_compression.rs (KvCompressionConfig :73-98, validate :123-172, validate_runtime_support :174-241).
// Same field names, defaults, accepted combinations and error texts, so a host that already drives the
// reference finds the same contract here.
#pragma once
#include <stdint.h>

#include <string>

namespace m40host {

enum class KvCompressMode : uint32_t { Off = 0, DenseRecentOnly, RecentOnly, BlockSummary, BlockSelectLossy, BlockSelectExact };
enum class KvRepresentativePolicy : uint32_t { Last = 0, Spread = 1 };
enum class KvExactOldBacking : uint32_t { Dense = 0, Q8 = 1, Fp16KQ4V = 2 };
enum class KvExactOldAttention : uint32_t { Staged = 0, Q8Direct = 1, Fp16KQ4VDirect = 2 };

const char* to_string(KvExactOldBacking b);
const char* to_string(KvExactOldAttention a);

struct KvCompressionConfig {
    KvCompressMode mode = KvCompressMode::BlockSelectExact;
    uint32_t recent_window = 1024;
    uint32_t block_size = 32;
    uint32_t top_blocks = 8;
    uint32_t representatives = 0;
    KvRepresentativePolicy representative_policy = KvRepresentativePolicy::Last;
    KvExactOldBacking exact_old_backing = KvExactOldBacking::Fp16KQ4V;
    KvExactOldAttention exact_old_attention = KvExactOldAttention::Fp16KQ4VDirect;

    static KvCompressionConfig dense_reference();
    static KvCompressionConfig for_mode(KvCompressMode mode);

    // Empty string = valid; otherwise the reference's error message.
    std::string validate() const;
    std::string validate_runtime_support(uint32_t max_seq_len, uint32_t head_dim) const;
    // What this B200 library can execute: Off, or BlockSelectExact with the FP16-K/q4-V direct path.
    std::string validate_b200_support(uint32_t max_seq_len, uint32_t head_dim) const;
};

}  // namespace m40host
