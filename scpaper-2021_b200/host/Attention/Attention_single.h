// The reference's Attention/Attention_single.h is an empty include guard that its drivers and
// Encoder.h include (test/Encoder/test_sparsity.cu:2, Encoder/Encoder.h:8); the fused-QKV
// attention operator it once announced is the isSingleKernel specialisation in Attention.h.
#ifndef ATTN_SINGLE
#define ATTN_SINGLE
#include "Attention.h"
#endif
