/* Drives the reference's own samplers (tq_sample_argmax, tq_sample_topp; src/engine/tq_generate.c:30-40,
 * 81-156) on logits drawn from a xorshift generator and writes the tokens they pick: the anchor for
 * sample_argmax and sample_top_p in tests/plain/qwen2_moe_plain.py.
 *
 * samples.bin: int32 tokens, case after case in the order of the loops below; for each case the argmax
 * first, then DRAWS tokens of one generator state that starts at 1000 + the case's number.
 * tests/test_golden.py regenerates the logits and the reference's uniform numbers (its xorshift64*,
 * :53-58) and asks the plain sampler for the same draws.  Built and run by make_golden.sh.
 */
#include "turboquant/tq_engine.h"
#include <stdio.h>
#include <stdlib.h>

#define DRAWS 24
static unsigned long long s = 88172645463325252ULL;
static float rnd(void) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return (float)(s >> 40) / (float)(1 << 24) - 0.5f; }

int main(void) {
    const int vocab[3] = {256, 1000, 5003};
    const float spread[3] = {4.0f, 10.0f, 25.0f};          /* logits in [-spread/2, spread/2) */
    const float temperature[3] = {0.7f, 1.0f, 0.3f};
    const float top_p[3] = {0.9f, 1.0f, 0.5f};
    FILE* O = fopen("samples.bin", "wb");
    int n_case = 0;
    for (int v = 0; v < 3; v++) {
        float* logits = malloc(vocab[v] * sizeof(float));
        for (int sp = 0; sp < 3; sp++) {
            for (int i = 0; i < vocab[v]; i++) logits[i] = rnd() * spread[sp];
            for (int t = 0; t < 3; t++)
                for (int p = 0; p < 3; p++, n_case++) {
                    int tok = tq_sample_argmax(logits, vocab[v]);
                    fwrite(&tok, 4, 1, O);
                    unsigned long long rng = 1000ULL + (unsigned long long)n_case;
                    for (int d = 0; d < DRAWS; d++) {
                        tok = tq_sample_topp(logits, vocab[v], temperature[t], top_p[p], &rng);
                        fwrite(&tok, 4, 1, O);
                    }
                }
        }
        free(logits);
    }
    fclose(O);
    printf("%d cases\n", n_case);
    return 0;
}
