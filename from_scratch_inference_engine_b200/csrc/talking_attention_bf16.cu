// The mixed-heads attention for bfloat16 pages (the kernels are in talking_attention.cuh).
#include "talking_attention.cuh"

extern "C" int fsie_talking_attention_bf16(fsie::TalkingArgs args, int num_tiles, cudaStream_t stream) {
    return fsie::talking_attention_launch<fsie::bf16>(args, num_tiles, stream);
}
