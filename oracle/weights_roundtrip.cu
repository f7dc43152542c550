// weights_roundtrip.cu: reads a weights.bin file with the REFERENCE's reader and writes it back
// with the reference's writer (cuda/weights.cu), as float32 or float16, so a test can prove that
// a file written by cuda_transformer_b200/weights.py is one every program of the reference
// loads, and that the fp16 file of this library equals the reference's own fp16 export.
// TEST INFRASTRUCTURE: linked by oracle/build_ref_tests.py against the reference's objects.
// Host code only; runs without a GPU.
#include <cstdio>
#include <cstring>
#include <string>

#include "weights.h"        // reference

int main(int argc, char *argv[])
{
    if (argc != 4 || (strcmp(argv[3], "f32") != 0 && strcmp(argv[3], "f16") != 0))
    {
        fprintf(stderr, "usage: weights_roundtrip in.bin out.bin f32|f16\n");
        return 2;
    }
    Weights w = read_weights(argv[1]);      // exits with a message if the file is bad
    printf("V %d Vp %d n_ctx %d L %d H %d C %d n %zu\n", w.cfg.V, w.cfg.Vp, w.cfg.n_ctx, w.cfg.L, w.cfg.H, w.cfg.C,
           w.params.size());
    write_weights(argv[2], w.cfg, w.params, strcmp(argv[3], "f16") == 0);
    return 0;
}
