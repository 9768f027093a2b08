// The attention kernel for variable-length batches: attn.cu compiled a second time with per-sequence offsets
// and lengths (cu_seqlens), see the note at the top of attn.cu.
#define SAGE3_VARLEN_BUILD 1
#include "attn.cu"
