// End-to-end driver around the REFERENCE engine's own Model and Transformer classes
// (src/model.cpp, src/transformer.cpp, compiled unmodified).  TEST INFRASTRUCTURE: built by
// oracle/Makefile twice --
//   _ref/engine_ref   with the reference's own ternary kernels,
//   _ref/engine_tllm  with libtllm_b200.so in their place (-DUSE_TLLM_B200), plus the
//                     load-time hook: every ternary matrix is repacked and registered,
//                     so the reference's unchanged call sites reach the fast kernels.
// It replaces the reference's src/main.cpp raw-token loop (main.cpp:282-359), which cannot be
// built here because it pulls in the SentencePiece tokenizer: seeded random prompt ids, one
// prefill forward, then greedy decode steps with the argmax taken on the host.
//
//   engine_xxx model.tllm n_prompt n_decode [logits_out.bin]
// prints one line:  prefill_ms=.. decode_ms=.. tok_per_s=.. last_token=..
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "model.h"
#include "transformer.h"
#ifdef USE_TLLM_B200
#include "tllm_b200.h"
#endif

#ifdef USE_TLLM_B200
static std::vector<void*> g_packed;
static void prepare(TernaryWeight& w, int gs)
{
    if (!w.nonzero_masks) return;
    const size_t bytes = tllm_b200_packed_bytes(w.out_features, w.in_features);
    void* packed = nullptr;
    if (!bytes || cudaMalloc(&packed, bytes) != cudaSuccess) return;
    const int st = tllm_b200_weight_prepare(w.nonzero_masks, w.sign_masks, w.scales, w.out_features,
                                            w.in_features, gs, packed, bytes, nullptr);
    if (st == TLLM_OK) {
        tllm_b200_weight_register(w.nonzero_masks, packed, w.out_features, w.in_features);
        g_packed.push_back(packed);
    } else {
        fprintf(stderr, "[engine] prepare failed (%s): %s\n", tllm_b200_status_string(st), tllm_b200_last_error());
        cudaFree(packed);
    }
}
#endif

static int argmax_host(const half* logits_gpu, int vocab, std::vector<half>& host)
{
    cudaMemcpy(host.data(), logits_gpu, (size_t)vocab * sizeof(half), cudaMemcpyDeviceToHost);
    int best = 0;
    float bv = -1e30f;
    for (int i = 0; i < vocab; i++) {
        const float v = __half2float(host[i]);
        if (v > bv) { bv = v; best = i; }
    }
    return best;
}

int main(int argc, char** argv)
{
    if (argc < 4) {
        fprintf(stderr, "usage: %s model.tllm n_prompt n_decode [logits_out.bin]\n", argv[0]);
        return 2;
    }
    const int n_prompt = atoi(argv[2]), n_decode = atoi(argv[3]);
    Model model = Model::load(argv[1]);
    const int gs = (int)model.config.group_size;
#ifdef USE_TLLM_B200
    for (auto& l : model.layers) {
        prepare(l.q_proj, gs); prepare(l.k_proj, gs); prepare(l.v_proj, gs); prepare(l.o_proj, gs);
        prepare(l.gate_proj, gs); prepare(l.up_proj, gs); prepare(l.down_proj, gs);
    }
    if (model.lm_head_is_ternary) prepare(model.lm_head_ternary, gs);
    fprintf(stderr, "[engine] %zu matrices prepared for libtllm_b200\n", g_packed.size());
#else
    (void)gs;
#endif
    Transformer tf(model);
    const int vocab = (int)model.config.vocab_size;
    std::mt19937 rng(1234);
    std::vector<int> prompt(n_prompt);
    for (auto& t : prompt) t = (int)(rng() % (unsigned)vocab);
    int* tok_gpu = nullptr;
    cudaMalloc(&tok_gpu, sizeof(int) * (size_t)(n_prompt > 1 ? n_prompt : 1));
    cudaMemcpy(tok_gpu, prompt.data(), sizeof(int) * (size_t)n_prompt, cudaMemcpyHostToDevice);
    std::vector<half> host((size_t)vocab);

    auto t0 = std::chrono::steady_clock::now();
    half* logits = tf.forward(tok_gpu, n_prompt, 0);
    cudaDeviceSynchronize();
    auto t1 = std::chrono::steady_clock::now();
    int tok = argmax_host(logits, vocab, host);
    int pos = n_prompt;
    auto t2 = std::chrono::steady_clock::now();
    for (int i = 0; i < n_decode; i++) {
        cudaMemcpy(tok_gpu, &tok, sizeof(int), cudaMemcpyHostToDevice);
        logits = tf.forward(tok_gpu, 1, pos++);
        cudaDeviceSynchronize();
        tok = argmax_host(logits, vocab, host);
    }
    auto t3 = std::chrono::steady_clock::now();
    const double prefill_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    const double decode_ms = std::chrono::duration<double, std::milli>(t3 - t2).count();
    if (argc > 4) {
        FILE* f = fopen(argv[4], "wb");
        if (f) { fwrite(host.data(), sizeof(half), (size_t)vocab, f); fclose(f); }
    }
    const cudaError_t e = cudaGetLastError();
    printf("prefill_ms=%.3f decode_ms=%.3f tok_per_s=%.2f last_token=%d cuda=%s\n", prefill_ms, decode_ms,
           n_decode > 0 ? n_decode * 1e3 / decode_ms : 0.0, tok, cudaGetErrorString(e));
    return e == cudaSuccess ? 0 : 1;
}
