// Attention whose heads talk before the softmax, bfloat16 storage.
#include "attention_talking.cuh"

KVF_TALK_API(bf16, bf16)
