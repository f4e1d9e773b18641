/* Times the reference's own CPU forward (tq_forward, one token of one sequence at a time) on an in-memory model
 * with the layer sizes of Qwen1.5-MoE-A2.7B: hidden 2048, 16 heads x 128, 60 experts top-4 of 1408, shared expert
 * 5632, vocabulary 151,936, all weights float32, L layers (argument 1) and T threads (argument 2).  The model is
 * built by hand as ref_driver.c builds its tiny one.  After 4 warm-up tokens it times 16 tokens at positions 4..19
 * and prints the mean milliseconds per token.  Run for L = 1 and L = 2 the difference is the cost of one layer, and
 * the cost of the 24-layer model follows (time_reference.sh does that and writes reference_cpu_timing.txt).
 * The reference has no batch and no prompt step for this architecture (src/engine/tq_transformer.c:3066-3067), so
 * this token-by-token rate is both its decode and its prefill speed.
 */
#include "turboquant/tq_engine.h"
#include "turboquant/tq_gguf.h"
#include "turboquant/turboquant.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

static unsigned long long s = 88172645463325252ULL;
static float rnd(void) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return ((float)(s >> 40) / (float)(1 << 24) - 0.5f) * 0.07f; }
static float* fill(size_t n) { float* p = malloc(n * sizeof(float)); for (size_t i = 0; i < n; i++) p[i] = rnd(); return p; }
static float* ones(size_t n) { float* p = malloc(n * sizeof(float)); for (size_t i = 0; i < n; i++) p[i] = 1.0f + rnd() * 0.1f; return p; }
static double now(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }

int main(int argc, char** argv) {
    int L = argc > 1 ? atoi(argv[1]) : 1, threads = argc > 2 ? atoi(argv[2]) : 8;
    tq_model_t m; memset(&m, 0, sizeof m); tq_model_config_t* c = &m.config;
    int D = 2048, NH = 16, NKV = 16, HD = 128, E = 60, K = 4, I = 1408, S = 5632, V = 151936; int Q = NH * HD, KV = NKV * HD;
    c->n_layers = L; c->hidden_dim = D; c->n_heads = NH; c->n_kv_heads = NKV; c->head_dim = HD; c->vocab_size = V; c->max_seq_len = 64;
    c->rope_freq_base = 1000000.f; c->rms_norm_eps = 1e-6f; c->is_moe = 1; c->num_experts = E; c->num_active_experts = K;
    c->expert_intermediate_dim = I; c->has_shared_expert = 1; c->shared_expert_intermediate_dim = S; c->intermediate_dim = S; c->model_type = 2;
    tq_moe_config_t mc; memset(&mc, 0, sizeof mc); mc.num_experts = E; mc.num_active = K; mc.expert_intermediate_dim = I;
    mc.has_shared_expert = 1; mc.shared_expert_intermediate_dim = S; mc.norm_topk_prob = 1;
    m.moe_config = &mc;
    m.token_embedding = fill((size_t)V * D); m.output_weight = fill((size_t)V * D); m.output_norm = ones(D);
    m.layers = calloc(L, sizeof(tq_layer_weights_t));
    for (int l = 0; l < L; l++) {
        tq_layer_weights_t* Y = &m.layers[l];
        Y->attn_norm = ones(D); Y->ffn_norm = ones(D); Y->wq = fill((size_t)Q * D); Y->wk = fill((size_t)KV * D);
        Y->wv = fill((size_t)KV * D); Y->wo = fill((size_t)D * Q);
        Y->q_bias = fill(Q); Y->k_bias = fill(KV); Y->v_bias = fill(KV);
        tq_moe_layer_t* ml = calloc(1, sizeof *ml); ml->router_weight = fill((size_t)E * D); ml->experts = calloc(E, sizeof(tq_expert_weights_t));
        for (int e = 0; e < E; e++) {
            ml->experts[e].w_gate = fill((size_t)I * D); ml->experts[e].w_up = fill((size_t)I * D); ml->experts[e].w_down = fill((size_t)D * I);
            ml->experts[e].gate_type = ml->experts[e].up_type = ml->experts[e].down_type = TQ_GGML_TYPE_F32;
        }
        ml->shared_expert.w_gate = fill((size_t)S * D); ml->shared_expert.w_up = fill((size_t)S * D); ml->shared_expert.w_down = fill((size_t)D * S);
        ml->shared_expert.gate_type = ml->shared_expert.up_type = ml->shared_expert.down_type = TQ_GGML_TYPE_F32;
        ml->shared_gate = fill(D); Y->moe = ml;
    }
    tq_set_threads(threads);
    tq_state_t* st = tq_create_state(c, TQ_TYPE_COUNT); st->moe_state = tq_moe_create_state(&mc, D);
    int tok = 3; float* lg = NULL;
    for (int i = 0; i < 4; i++) { lg = tq_forward(&m, st, tok, i); tok = (tok * 7919 + 13) % V; }
    double t0 = now();
    for (int i = 4; i < 20; i++) { lg = tq_forward(&m, st, tok, i); tok = (tok * 7919 + 13) % V; }
    double ms = (now() - t0) * 1e3 / 16;
    printf("layers %d threads %d ms_per_token %.3f (a logit: %g)\n", L, threads, ms, lg[0]);
    return 0;
}
