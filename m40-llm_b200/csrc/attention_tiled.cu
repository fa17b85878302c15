// Tiled decode attention for head_dim 64/128 (placeholder until the tensor-core kernel lands).
#include "attention.cuh"
int m40_attention_dense_tiled(M40llmCudaContext*, const DenseAttnArgs&, uint32_t) { return 1; }
