// The persistent Llama decode-step kernel once more, with a poll limit of a few milliseconds instead of two seconds: the build
// pt_llama_decode_step launches when pt_llama_step_args.wait_limit is non-zero (tests of the bounded-wait path, hosts that prefer
// a quick failure).  The limit stays a compile-time constant in both builds.
#define PT_MK_SHORT_VARIANT
#include "decode_llama.cu"
