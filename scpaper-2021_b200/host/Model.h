// Shape record shared by the attention and encoder operators.
// Same leading fields, in the same order, as the reference's Model_t (Model.h:2-10), so
// `Model_t{768, 768, 128, 12, 3072, 768}` keeps compiling.  Two trailing fields are new:
// the reference has no batch dimension and hard-codes a causal mask (Attention.h:97-104).
#pragma once
struct Model_t {
    int kdim;     // total Q/K width (nhead * head dim)
    int vdim;     // total V width
    int seq_len;  // tokens per sequence
    int nhead;
    int dimFF;
    int emdim;  // model width
    int nlayer = 1;
    int batch = 1;      // sequences per forward call; every operator works on batch * seq_len rows
    int mask_kind = 1;  // ET_MASK_CAUSAL, the reference default; 0 none, 2 padding, 3 additive
};
