/* A second run of the reference's own CPU model code for what ref_driver.c leaves out:
 *   - a dense SwiGLU layer in a model with experts (layer 1 has no router: `moe` is NULL and w_gate/w_up/w_down are
 *     set, src/engine/tq_transformer.c:2707-2824), after a layer with experts (layer 0);
 *   - a tied head (output_weight is the embedding table, src/engine/tq_model.c:1499-1516);
 *   - the router alone (tq_moe_route, src/engine/tq_moe.c:600-682): ids and weights of the 3 largest of 8 logits
 *     for 6 hidden vectors.
 * Weights come from the same xorshift generator as in ref_driver.c, in creation order; tests/test_golden.py draws
 * the same numbers.  Writes logits2.bin (7 positions x 256 logits, float32) and route.bin (6 x 3 int32 ids, then
 * 6 x 3 float32 weights).  Built and run by make_golden.sh.
 */
#include "turboquant/tq_engine.h"
#include "turboquant/tq_gguf.h"
#include "turboquant/turboquant.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static unsigned long long s = 88172645463325252ULL;
static float rnd(void) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return ((float)(s >> 40) / (float)(1 << 24) - 0.5f) * 0.2f; }
static float* fill(size_t n) { float* p = malloc(n * sizeof(float)); for (size_t i = 0; i < n; i++) p[i] = rnd(); return p; }
static float* ones(size_t n) { float* p = malloc(n * sizeof(float)); for (size_t i = 0; i < n; i++) p[i] = 1.0f + rnd() * 0.1f; return p; }

int main(void) {
    tq_model_t m; memset(&m, 0, sizeof m); tq_model_config_t* c = &m.config;
    int L = 2, D = 64, NH = 4, NKV = 2, HD = 16, E = 8, K = 2, I = 32, S = 64, ID = 80, V = 256; int Q = NH * HD, KV = NKV * HD;
    c->n_layers = L; c->hidden_dim = D; c->n_heads = NH; c->n_kv_heads = NKV; c->head_dim = HD; c->vocab_size = V; c->max_seq_len = 128;
    c->rope_freq_base = 10000.f; c->rms_norm_eps = 1e-6f; c->is_moe = 1; c->num_experts = E; c->num_active_experts = K;
    c->expert_intermediate_dim = I; c->has_shared_expert = 1; c->shared_expert_intermediate_dim = S; c->intermediate_dim = ID; c->model_type = 2;
    tq_moe_config_t mc; memset(&mc, 0, sizeof mc); mc.num_experts = E; mc.num_active = K; mc.expert_intermediate_dim = I;
    mc.has_shared_expert = 1; mc.shared_expert_intermediate_dim = S; mc.norm_topk_prob = 1;
    m.moe_config = &mc;
    m.token_embedding = fill((size_t)V * D); m.output_weight = m.token_embedding; m.output_norm = ones(D);      /* tied */
    m.layers = calloc(L, sizeof(tq_layer_weights_t));
    for (int l = 0; l < L; l++) {
        tq_layer_weights_t* Y = &m.layers[l];
        Y->attn_norm = ones(D); Y->ffn_norm = ones(D); Y->wq = fill(Q * D); Y->wk = fill(KV * D); Y->wv = fill(KV * D); Y->wo = fill(D * Q);
        Y->q_bias = fill(Q); Y->k_bias = fill(KV); Y->v_bias = fill(KV);
        if (l == 1) {                                                      /* the dense layer */
            Y->w_gate = fill((size_t)ID * D); Y->w_up = fill((size_t)ID * D); Y->w_down = fill((size_t)D * ID);
            continue;
        }
        tq_moe_layer_t* ml = calloc(1, sizeof *ml); ml->router_weight = fill(E * D); ml->experts = calloc(E, sizeof(tq_expert_weights_t));
        for (int e = 0; e < E; e++) {
            ml->experts[e].w_gate = fill(I * D); ml->experts[e].w_up = fill(I * D); ml->experts[e].w_down = fill(D * I);
            ml->experts[e].gate_type = ml->experts[e].up_type = ml->experts[e].down_type = TQ_GGML_TYPE_F32;
        }
        ml->shared_expert.w_gate = fill(S * D); ml->shared_expert.w_up = fill(S * D); ml->shared_expert.w_down = fill(D * S);
        ml->shared_expert.gate_type = ml->shared_expert.up_type = ml->shared_expert.down_type = TQ_GGML_TYPE_F32;
        ml->shared_gate = fill(D); Y->moe = ml;
    }
    tq_state_t* st = tq_create_state(c, TQ_TYPE_COUNT); st->moe_state = tq_moe_create_state(&mc, D);
    int toks[7] = {3, 17, 200, 42, 9, 77, 255}; FILE* O = fopen("logits2.bin", "wb");
    for (int i = 0; i < 7; i++) { float* lg = tq_forward(&m, st, toks[i], i); fwrite(lg, 4, V, O); }
    fclose(O);
    /* the router alone */
    float* wr = fill((size_t)E * D); float* hid = fill((size_t)6 * D);
    int ids[18]; float wts[18];
    for (int t = 0; t < 6; t++) tq_moe_route(hid + (size_t)t * D, wr, E, 3, D, ids + 3 * t, wts + 3 * t);
    O = fopen("route.bin", "wb"); fwrite(ids, 4, 18, O); fwrite(wts, 4, 18, O); fclose(O);
    puts("done");
    return 0;
}
