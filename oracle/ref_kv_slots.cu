// TEST INFRASTRUCTURE ONLY.  Prints KVBlockArray::getKVTokenIdx of the reference's own header
// (cpp/tensorrt_llm/kernels/kvCacheUtils.h, compiled from the reference tree where it lies) for one parameter
// set: the slot of every token index 0 .. ntok-1 and the constants the constructor derived.  Used once, by
// tests/golden/make_golden.py, to write tests/golden/kv_slot_golden.json; nothing at run time depends on it.
//   ref_kv_slots <tokens_per_block> <max_blocks_per_seq> <attention_window> <sink_tokens> <ntok>
#include <cstdio>
#include <cstdlib>

#include "tensorrt_llm/kernels/kvCacheUtils.h"

int main(int argc, char** argv)
{
    if (argc != 6)
        return 2;
    const int tpb = atoi(argv[1]), m = atoi(argv[2]), window = atoi(argv[3]), sink = atoi(argv[4]), ntok = atoi(argv[5]);
    tensorrt_llm::kernels::KVBlockArray arr(1, m, tpb, 1, window, sink, false);
    printf("{\"tokens_per_block\": %d, \"max_blocks_per_seq\": %d, \"attention_window\": %d, \"sink_tokens\": %d, "
           "\"bubble_len\": %d, \"cyclic_cache_len\": %d, \"one_more_block\": %d, \"slots\": [",
        tpb, m, window, sink, (int) arr.mBubbleLen, (int) arr.mCyclicCacheLen, (int) arr.mEnableOneMoreBlock);
    for (int t = 0; t < ntok; ++t)
        printf("%s%d", t ? ", " : "", (int) arr.getKVTokenIdx(t));
    printf("]}\n");
    return 0;
}
