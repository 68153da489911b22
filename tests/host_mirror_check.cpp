// Compile-and-link check of the C++ host mirror against libdecode_attn.so; prints struct sizes so
// that the ctypes declarations can be compared with the C layout.  Launches nothing.
#include <cstdio>
#include <cstring>

#include "gpt_attention_common.h"

int main(int argc, char** argv)
{
    std::printf("abi=%d config=%zu params=%zu\n", dx_abi_version(), sizeof(dx_attn_config),
        sizeof(dx_attn_generation_params));
    dx::GPTAttentionCommon op(0, 8, 2, 128, 1.f, 1, 0, true, true, DX_QUANT_FP8_KV_CACHE, true, 64, DX_DTYPE_BF16, 0);
    dx::EnqueueGenerationParams<uint16_t> p;
    // without initialize() the call must be refused on the host
    const int st = op.enqueueGeneration(p, nullptr);
    std::printf("uninitialised enqueue -> %s\n", dx_strerror(st));
    if (argc > 1 && !std::strcmp(argv[1], "--init"))
        std::printf("initialize -> %s\n", dx_strerror(op.initialize()));
    return st == DX_ERR_BAD_ARG ? 0 : 1;
}
