// ckpt_roundtrip.cu: reads a GPTC checkpoint with the REFERENCE's reader and writes it back
// with the reference's writer (cuda/checkpoint.cu), so a test can prove that a file written by
// cuda_transformer_b200/checkpoint.py is one the reference resumes from, byte for byte.
// TEST INFRASTRUCTURE: linked by oracle/build_ref_tests.py against the reference's objects.
// Host code only; runs without a GPU.
#include <cstdio>
#include <string>

#include "checkpoint.h"     // reference

int main(int argc, char *argv[])
{
    if (argc != 3)
    {
        fprintf(stderr, "usage: ckpt_roundtrip in.ckpt out.ckpt\n");
        return 2;
    }
    Checkpoint c;
    std::string why;
    if (!try_read_checkpoint(argv[1], c, why))
    {
        fprintf(stderr, "the reference's reader rejects %s: %s\n", argv[1], why.c_str());
        return 1;
    }
    printf("V %d Vp %d n_ctx %d L %d H %d C %d step %d adam_t %d loss_scale %g n %zu keep '%s'\n", c.cfg.V, c.cfg.Vp,
           c.cfg.n_ctx, c.cfg.L, c.cfg.H, c.cfg.C, c.state.step, c.state.adam_t, c.state.loss_scale, c.params.size(),
           c.run.keep.c_str());
    write_checkpoint(argv[2], c);
    return 0;
}
