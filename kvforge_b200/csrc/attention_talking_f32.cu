// Attention whose heads talk before the softmax, 32-bit storage.
#include "attention_talking.cuh"

KVF_TALK_API(f32, float)
