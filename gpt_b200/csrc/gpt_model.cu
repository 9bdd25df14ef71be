// GptModel: host-side driver of one GPT-2 training / inference step over an IGPTBackend.
//
// It issues the operator sequence of the reference's model class (src/model/gpt.cpp:426-642: embedding,
// per layer LN1 -> QKV -> attention -> projection -> LN2 -> FFN up (GELU) -> FFN down, final LN, un-embedding,
// softmax; and the mirror image for the backward pass) and keeps the reference's parameter packing
// (src/model/gpt.cpp:46-62: sixteen tensors, kind-major, all layers of a kind contiguous, no padding), so raw
// fp32 checkpoints of the reference load unchanged and gradient buffers compare element for element.
//
// What is added for data-parallel training: the backward pass can report, layer by layer, that the weight
// gradients of a layer are complete (a host callback fired right after that layer's operators were enqueued),
// so that the caller can start all-reducing finished slices on another stream while the remaining layers run.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "backend_interface.h"
#include "b200_backend.h"
#include "../../include/gptb200.h"

namespace {

struct Config {
    int max_seq_len, vocab, vocab_padded, layers, heads, d_model, d_ffn;
};

// Offsets (in floats) of the sixteen parameter tensors inside one packed buffer.
struct ParamLayout {
    size_t wte, wpe, ln1_w, ln1_b, qkv_w, qkv_b, proj_w, proj_b, ln2_w, ln2_b, up_w, up_b, down_w, down_b, lnf_w, lnf_b, total;
    explicit ParamLayout(const Config &c)
    {
        const size_t L = c.layers, D = c.d_model, F = c.d_ffn;
        size_t o = 0;
        auto take = [&](size_t n) { const size_t at = o; o += n; return at; };
        wte = take(size_t(c.vocab_padded) * D);
        wpe = take(size_t(c.max_seq_len) * D);
        ln1_w = take(L * D);
        ln1_b = take(L * D);
        qkv_w = take(L * D * 3 * D);
        qkv_b = take(L * 3 * D);
        proj_w = take(L * D * D);
        proj_b = take(L * D);
        ln2_w = take(L * D);
        ln2_b = take(L * D);
        up_w = take(L * D * F);
        up_b = take(L * F);
        down_w = take(L * F * D);
        down_b = take(L * D);
        lnf_w = take(D);
        lnf_b = take(D);
        total = o;
    }
};

size_t pad4(size_t n) { return (n + 3) & ~size_t(3); }

class GptModel
{
public:
    GptModel(IGPTBackend *be, const Config &c, bool use_grad) : be_(be), c_(c), lay_(c), use_grad_(use_grad)
    {
        const int nbuf = use_grad ? 4 : 1;  // weights, gradients, Adam first and second moments
        for (int i = 0; i < nbuf; ++i) {
            void *p = nullptr;
            be_->device_malloc(&p, lay_.total * sizeof(float));
            be_->device_memset(p, 0, lay_.total * sizeof(float));
            bufs_[i] = static_cast<float *>(p);
        }
        void *l = nullptr;
        be_->device_malloc(&l, sizeof(float));
        loss_dev_ = static_cast<float *>(l);
    }

    ~GptModel()
    {
        release_activations();
        for (float *b : bufs_)
            if (b) be_->device_free(b);
        if (loss_dev_) be_->device_free(loss_dev_);
    }

    float *weights() { return bufs_[0]; }
    float *grads() { return bufs_[1]; }
    size_t num_params() const { return lay_.total; }
    const ParamLayout &layout() const { return lay_; }

    // Same initialisation as the reference (src/model/gpt.cpp:297-325: the residual projections are drawn with mean 0
    // whatever `mean` is) plus zeroed padding rows of wte (the reference leaves them normal-filled; zero rows give exactly
    // zero logits and gradients in the padding columns).
    void init(float mean, float stddev)
    {
        float *w = weights();
        const size_t L = c_.layers, D = c_.d_model, F = c_.d_ffn;
        be_->device_fill_normal(w, mean, stddev, lay_.total);
        const float resid = stddev / sqrtf(2.0f * c_.layers);
        be_->device_fill_normal(w + lay_.proj_w, 0.0f, resid, L * D * D);
        be_->device_fill_normal(w + lay_.down_w, 0.0f, resid, L * F * D);
        for (size_t off : {lay_.ln1_w, lay_.ln2_w}) be_->device_fill_const(w + off, 1.0f, L * D);
        be_->device_fill_const(w + lay_.lnf_w, 1.0f, D);
        for (size_t off : {lay_.ln1_b, lay_.proj_b, lay_.ln2_b, lay_.down_b}) be_->device_fill_const(w + off, 0.0f, L * D);
        be_->device_fill_const(w + lay_.qkv_b, 0.0f, L * 3 * D);
        be_->device_fill_const(w + lay_.up_b, 0.0f, L * F);
        be_->device_fill_const(w + lay_.lnf_b, 0.0f, D);
        be_->device_fill_const(w + lay_.wte + size_t(c_.vocab) * D, 0.0f, size_t(c_.vocab_padded - c_.vocab) * D);
    }

    // Unlike the reference (src/model/gpt.cpp:399-424 frees and reallocates on every call, i.e. once per generated
    // token in its inference loop), buffers are kept when the new shape fits into what is already allocated.
    // Returns false when memory for the new shape cannot be had: the model then keeps its previous shape and buffers.
    bool set_size(int batch, int seq)
    {
        const size_t M = size_t(batch) * seq, L = c_.layers, D = c_.d_model, F = c_.d_ffn, H = c_.heads, Vp = c_.vocab_padded;
        size_t o = 0;
        auto take = [&](size_t n) { const size_t at = o; o += pad4(n); return at; };
        ActLayout a{};
        a.x_emb = take(M * D);
        a.ln1 = take(L * M * D); a.ln1_mean = take(L * M); a.ln1_var = take(L * M);
        a.qkv = take(L * M * 3 * D); a.lse = take(L * M * H); a.attn = take(L * M * D); a.proj = take(L * M * D);
        a.ln2 = take(L * M * D); a.ln2_mean = take(L * M); a.ln2_var = take(L * M);
        a.up = take(L * M * F); a.act = take(L * M * F); a.down = take(L * M * D);
        a.lnf = take(M * D); a.lnf_mean = take(M); a.lnf_var = take(M);
        // fused cross-entropy: the logits become their own gradient in place; only the row terms of the loss are kept
        const bool fused = fused_ce_ && use_grad_ && ctx_ != nullptr;
        a.logits = take(M * Vp); a.probs = fused ? a.logits : take(M * Vp);
        a.row_loss = take(fused ? M : 0);
        a.total = o;
        GradLayout g{};
        if (use_grad_) {
            // activation gradients are consumed right after they are produced: one set of buffers serves all layers
            o = 0;
            g.d_ln = take(M * D); g.d_res = take(M * D); g.d_x = take(M * D); g.d_qkv = take(M * 3 * D); g.d_helper = take(M * H);
            g.d_f1 = take(M * F); g.d_f2 = take(M * F); g.d_logits = take(fused ? 0 : M * Vp);
            g.total = o;
        }
        // the new buffers first: if one cannot be had, nothing has changed
        void *new_acts = nullptr, *new_grads = nullptr;
        const bool need_acts = a.total > acts_capacity_, need_grads = use_grad_ && g.total > agrads_capacity_;
        if (need_acts) be_->device_malloc(&new_acts, a.total * sizeof(float));
        if (need_grads) be_->device_malloc(&new_grads, g.total * sizeof(float));
        if ((need_acts && !new_acts) || (need_grads && !new_grads)) {   // a non-aborting backend leaves a null pointer
            if (new_acts) be_->device_free(new_acts);
            if (new_grads) be_->device_free(new_grads);
            return false;
        }
        if (new_acts) {
            if (acts_) be_->device_free(acts_);
            acts_ = static_cast<float *>(new_acts);
            acts_capacity_ = a.total;
        }
        if (new_grads) {
            if (agrads_) be_->device_free(agrads_);
            agrads_ = static_cast<float *>(new_grads);
            agrads_capacity_ = g.total;
        }
        a_ = a;
        g_ = g;
        fused_ce_active_ = fused;
        row_loss_valid_ = false;
        B_ = batch;
        T_ = seq;
        if (use_grad_) be_->device_memset(agrads_, 0, g_.total * sizeof(float));  // the padding columns of d_logits must be zero
        return true;
    }

    void zero_grad()
    {
        if (use_grad_) be_->device_memset(grads(), 0, lay_.total * sizeof(float));
    }

    void forward(const int *tokens)
    {
        const size_t M = size_t(B_) * T_, D = c_.d_model, F = c_.d_ffn, H = c_.heads;
        float *w = weights(), *A = acts_;
        be_->device_embedding_forward(A + a_.x_emb, w + lay_.wte, w + lay_.wpe, tokens, B_, T_, c_.d_model);
        float *stream = A + a_.x_emb;  // residual stream entering the next LayerNorm
        float *resid = nullptr;        // pending residual, added inside the next LayerNorm
        for (int l = 0; l < c_.layers; ++l) {
            float *ln1 = A + a_.ln1 + l * M * D, *qkv = A + a_.qkv + l * M * 3 * D, *attn = A + a_.attn + l * M * D;
            float *proj = A + a_.proj + l * M * D, *ln2 = A + a_.ln2 + l * M * D, *up = A + a_.up + l * M * F;
            float *act = A + a_.act + l * M * F, *down = A + a_.down + l * M * D;
            be_->device_layernorm_residual_fused_forward(ln1, A + a_.ln1_mean + l * M, A + a_.ln1_var + l * M, stream, resid, w + lay_.ln1_w + l * D,
                                                         w + lay_.ln1_b + l * D, B_, T_, c_.d_model);
            resid = stream;
            be_->device_linear_activation_fused_forward(qkv, nullptr, ln1, w + lay_.qkv_w + l * D * 3 * D, w + lay_.qkv_b + l * 3 * D, false, B_, T_,
                                                        c_.d_model, 3 * c_.d_model);
            be_->device_flash_attention_forward(attn, A + a_.lse + l * M * H, qkv, B_, T_, c_.d_model, c_.heads);
            be_->device_linear_activation_fused_forward(proj, nullptr, attn, w + lay_.proj_w + l * D * D, w + lay_.proj_b + l * D, false, B_, T_,
                                                        c_.d_model, c_.d_model);
            be_->device_layernorm_residual_fused_forward(ln2, A + a_.ln2_mean + l * M, A + a_.ln2_var + l * M, proj, resid, w + lay_.ln2_w + l * D,
                                                         w + lay_.ln2_b + l * D, B_, T_, c_.d_model);
            resid = proj;
            be_->device_linear_activation_fused_forward(up, act, ln2, w + lay_.up_w + l * D * F, w + lay_.up_b + l * F, true, B_, T_, c_.d_model,
                                                        c_.d_ffn);
            be_->device_linear_activation_fused_forward(down, nullptr, act, w + lay_.down_w + l * F * D, w + lay_.down_b + l * D, false, B_, T_,
                                                        c_.d_ffn, c_.d_model);
            stream = down;
        }
        be_->device_layernorm_residual_fused_forward(A + a_.lnf, A + a_.lnf_mean, A + a_.lnf_var, stream, resid, w + lay_.lnf_w, w + lay_.lnf_b, B_, T_,
                                                     c_.d_model);
        be_->device_unembedding_forward(A + a_.logits, A + a_.lnf, w + lay_.wte, B_, T_, c_.d_model, c_.vocab_padded);
        if (use_grad_ && !fused_ce_active_) be_->device_softmax_forward(A + a_.probs, A + a_.logits, B_, T_, c_.vocab, c_.vocab_padded);
        row_loss_valid_ = false;
    }

    // layer_done(l, user): gradients of layer l's twelve parameter tensors are complete (enqueued);
    // l == layers means "un-embedding and final LayerNorm done (wte still open)", l == -1 means "everything done".
    void backward(const int *tokens, const int *labels, void (*layer_done)(int, void *), void *user)
    {
        const size_t M = size_t(B_) * T_, D = c_.d_model, F = c_.d_ffn, H = c_.heads;
        float *w = weights(), *gw = grads(), *A = acts_, *G = agrads_;
        float *d_ln = G + g_.d_ln, *d_res = G + g_.d_res, *d_x = G + g_.d_x;
        float *d_logits = G + g_.d_logits;
        if (fused_ce_active_) {
            // softmax, its gradient and the loss terms in one pass, in place: the logits buffer now holds the gradient
            d_logits = A + a_.logits;
            if (gptb200_softmax_cross_entropy_inplace(ctx_, d_logits, A + a_.row_loss, labels, B_ * T_, c_.vocab, c_.vocab_padded) != 0) return;
            row_loss_valid_ = true;
        } else {
            // the padding columns of d_logits are never written by the cross-entropy backward: they stay zero from set_size
            be_->device_cross_entropy_softmax_fused_backward(d_logits, A + a_.probs, labels, B_, T_, c_.vocab, c_.vocab_padded);
        }
        be_->device_unembedding_backward(d_x, gw + lay_.wte, d_logits, A + a_.lnf, w + lay_.wte, B_, T_, c_.d_model, c_.vocab_padded);
        be_->device_layernorm_residual_fused_backward(d_res, gw + lay_.lnf_w, gw + lay_.lnf_b, d_x, nullptr, A + a_.down + (c_.layers - 1) * M * D,
                                                      A + a_.lnf_mean, A + a_.lnf_var, w + lay_.lnf_w, B_, T_, c_.d_model);
        if (layer_done) layer_done(c_.layers, user);
        // d_res holds the gradient of the residual stream at the output of layer l
        for (int l = c_.layers - 1; l >= 0; --l) {
            if (fused_gelu_ && ctx_) {
                // the down projection's two halves apart: grad_x comes out already multiplied by the GELU derivative
                if (gptb200_linear_backward_weights(ctx_, gw + lay_.down_w + l * F * D, gw + lay_.down_b + l * D, d_res, A + a_.act + l * M * F,
                                                    static_cast<int>(M), c_.d_ffn, c_.d_model) != 0 ||
                    gptb200_linear_backward_input_gelu(ctx_, G + g_.d_f2, d_res, w + lay_.down_w + l * F * D, A + a_.up + l * M * F, static_cast<int>(M),
                                                       c_.d_ffn, c_.d_model) != 0)
                    return;
            } else {
                be_->device_linear_backward(G + g_.d_f1, gw + lay_.down_w + l * F * D, gw + lay_.down_b + l * D, d_res, A + a_.act + l * M * F,
                                            w + lay_.down_w + l * F * D, B_, T_, c_.d_ffn, c_.d_model);
                be_->device_activation_backward(G + g_.d_f2, G + g_.d_f1, A + a_.up + l * M * F, B_, T_, c_.d_ffn);
            }
            be_->device_linear_backward(d_x, gw + lay_.up_w + l * D * F, gw + lay_.up_b + l * F, G + g_.d_f2, A + a_.ln2 + l * M * D,
                                        w + lay_.up_w + l * D * F, B_, T_, c_.d_model, c_.d_ffn);
            be_->device_layernorm_residual_fused_backward(d_ln, gw + lay_.ln2_w + l * D, gw + lay_.ln2_b + l * D, d_x, d_res, A + a_.proj + l * M * D,
                                                          A + a_.ln2_mean + l * M, A + a_.ln2_var + l * M, w + lay_.ln2_w + l * D, B_, T_, c_.d_model);
            // d_ln: gradient of the stream after the attention projection (+ residual)
            be_->device_linear_backward(d_x, gw + lay_.proj_w + l * D * D, gw + lay_.proj_b + l * D, d_ln, A + a_.attn + l * M * D,
                                        w + lay_.proj_w + l * D * D, B_, T_, c_.d_model, c_.d_model);
            be_->device_flash_attention_backward(G + g_.d_qkv, G + g_.d_helper, A + a_.lse + l * M * H, d_x, A + a_.attn + l * M * D,
                                                 A + a_.qkv + l * M * 3 * D, B_, T_, c_.d_model, c_.heads);
            be_->device_linear_backward(d_x, gw + lay_.qkv_w + l * D * 3 * D, gw + lay_.qkv_b + l * 3 * D, G + g_.d_qkv, A + a_.ln1 + l * M * D,
                                        w + lay_.qkv_w + l * D * 3 * D, B_, T_, c_.d_model, 3 * c_.d_model);
            const float *ln1_in = l == 0 ? A + a_.x_emb : A + a_.down + (l - 1) * M * D;
            be_->device_layernorm_residual_fused_backward(d_res, gw + lay_.ln1_w + l * D, gw + lay_.ln1_b + l * D, d_x, d_ln, ln1_in,
                                                          A + a_.ln1_mean + l * M, A + a_.ln1_var + l * M, w + lay_.ln1_w + l * D, B_, T_, c_.d_model);
            if (layer_done) layer_done(l, user);
        }
        if (defer_embedding_) return;   // the caller applies the rows of all ranks itself (see apply_embedding_grad)
        be_->device_embedding_backward(gw + lay_.wte, gw + lay_.wpe, d_res, tokens, B_, T_, c_.d_model);
        if (layer_done) layer_done(-1, user);
    }

    // ---- KV-cached generation ------------------------------------------------------------------------------------
    // Prefill: forward over the prompt, then every layer's keys and values into the cache.  Returns a gptb200_status.
    int generate_begin(gptb200_ctx *ctx, const int *prompt, int batch, int prompt_len, int max_len)
    {
        const size_t L = c_.layers, D = c_.d_model, F = c_.d_ffn, Vp = c_.vocab_padded;
        if (!set_size(batch, prompt_len)) return GPTB200_ERR_CUDA;
        const size_t cache_floats = L * size_t(batch) * max_len * 2 * D;
        const size_t step_floats = size_t(batch) * (D * 7 + 3 * D + 2 * F + 6) + 8;
        if (cache_floats + step_floats > gen_capacity_) {
            void *p = nullptr;
            be_->device_malloc(&p, (cache_floats + step_floats) * sizeof(float));
            if (!p) return GPTB200_ERR_CUDA;
            if (gen_) be_->device_free(gen_);
            gen_ = static_cast<float *>(p);
            gen_capacity_ = cache_floats + step_floats;
        }
        gen_batch_ = batch;
        gen_max_len_ = max_len;
        gen_pos_ = prompt_len;
        forward(prompt);
        const size_t M = size_t(batch) * prompt_len;
        for (size_t l = 0; l < L; ++l) {
            const int rc = gptb200_kv_cache_fill(ctx, gen_ + l * size_t(batch) * max_len * 2 * D, acts_ + a_.qkv + l * M * 3 * D, batch, prompt_len, max_len,
                                                 c_.d_model);
            if (rc) return rc;
        }
        gen_pos_off_ = cache_floats + step_floats - 8;
        be_->device_memcpy_h2d(gen_ + gen_pos_off_, &gen_pos_, sizeof(int));
        (void)Vp;
        return GPTB200_OK;
    }

    // One new position for every sequence: the forward pass of one row per sequence, attention against the cache.
    int generate_step(gptb200_ctx *ctx, const int *tokens, float *logits)
    {
        if (!gen_ || gen_pos_ >= gen_max_len_ || gen_pos_ >= c_.max_seq_len) return GPTB200_ERR_INVALID_ARG;
        const size_t L = c_.layers, D = c_.d_model, F = c_.d_ffn;
        const int b = gen_batch_;
        const size_t cache_floats = L * size_t(b) * gen_max_len_ * 2 * D;
        float *s = gen_ + cache_floats;
        auto take = [&](size_t n) { float *at = s; s += n; return at; };
        float *x = take(b * D), *ln = take(b * D), *qkv = take(b * 3 * D), *attn = take(b * D), *proj = take(b * D), *up = take(b * F),
              *act = take(b * F), *down = take(b * D), *x2 = take(b * D), *mean = take(b), *var = take(b);
        (void)x2;
        int *pos_dev = reinterpret_cast<int *>(gen_ + gen_pos_off_);
        float *w = weights();
        int rc = gptb200_embedding_decode(ctx, x, w + lay_.wte, w + lay_.wpe, tokens, pos_dev, b, c_.d_model);
        if (rc) return rc;
        // same operator sequence as forward() with one row per sequence; the residual stream alternates between x / proj / down
        float *stream = x, *resid = nullptr;
        for (size_t l = 0; l < L; ++l) {
            be_->device_layernorm_residual_fused_forward(ln, mean, var, stream, resid, w + lay_.ln1_w + l * D, w + lay_.ln1_b + l * D, b, 1, c_.d_model);
            resid = stream;
            be_->device_linear_activation_fused_forward(qkv, nullptr, ln, w + lay_.qkv_w + l * D * 3 * D, w + lay_.qkv_b + l * 3 * D, false, b, 1, c_.d_model,
                                                        3 * c_.d_model);
            rc = gptb200_attention_decode(ctx, attn, gen_ + l * size_t(b) * gen_max_len_ * 2 * D, qkv, pos_dev, b, gen_max_len_, c_.d_model, c_.heads);
            if (rc) return rc;
            float *pj = (resid == proj) ? x : proj;   // never overwrite the pending residual
            be_->device_linear_activation_fused_forward(pj, nullptr, attn, w + lay_.proj_w + l * D * D, w + lay_.proj_b + l * D, false, b, 1, c_.d_model,
                                                        c_.d_model);
            be_->device_layernorm_residual_fused_forward(ln, mean, var, pj, resid, w + lay_.ln2_w + l * D, w + lay_.ln2_b + l * D, b, 1, c_.d_model);
            resid = pj;
            be_->device_linear_activation_fused_forward(up, act, ln, w + lay_.up_w + l * D * F, w + lay_.up_b + l * F, true, b, 1, c_.d_model, c_.d_ffn);
            float *dn = (resid == down) ? x : down;
            be_->device_linear_activation_fused_forward(dn, nullptr, act, w + lay_.down_w + l * F * D, w + lay_.down_b + l * D, false, b, 1, c_.d_ffn,
                                                        c_.d_model);
            stream = dn;
        }
        be_->device_layernorm_residual_fused_forward(ln, mean, var, stream, resid, w + lay_.lnf_w, w + lay_.lnf_b, b, 1, c_.d_model);
        be_->device_unembedding_forward(logits, ln, w + lay_.wte, b, 1, c_.d_model, c_.vocab_padded);
        rc = gptb200_advance_position(ctx, pos_dev);
        if (rc) return rc;
        ++gen_pos_;
        return GPTB200_OK;
    }

    int generate_position() const { return gen_ ? gen_pos_ : -1; }

    void set_defer_embedding(bool on) { defer_embedding_ = on; }
    void set_context(gptb200_ctx *ctx) { ctx_ = ctx; }
    void set_fused_cross_entropy(bool on) { fused_ce_ = on; }
    void set_fused_gelu_backward(bool on) { fused_gelu_ = on; }
    float *embedding_grad() { return agrads_ ? agrads_ + g_.d_res : nullptr; }
    size_t wte_offset() const { return lay_.wte; }
    size_t wpe_offset() const { return lay_.wpe; }

    float loss(const int *labels)
    {
        if (fused_ce_active_) {
            // after a backward pass the row terms are there; before it they are computed from the (still untouched) logits
            if (row_loss_valid_)
                gptb200_row_loss_mean(ctx_, loss_dev_, acts_ + a_.row_loss, B_ * T_);
            else
                gptb200_cross_entropy_loss_from_logits(ctx_, loss_dev_, acts_ + a_.row_loss, acts_ + a_.logits, labels, B_ * T_, c_.vocab, c_.vocab_padded);
        } else {
            be_->device_cross_entropy_loss(loss_dev_, acts_ + a_.probs, labels, B_, T_, c_.vocab_padded);
        }
        float v = 0.0f;
        be_->device_memcpy_d2h(&v, loss_dev_, sizeof(float));
        return v;
    }

    void clip(float max_norm, int accum_steps) { be_->device_scale_and_clip_grad(grads(), static_cast<int>(lay_.total), max_norm, accum_steps); }

    // AdamW over the sixteen tensors; weight decay only on the matrices and embeddings (src/model/gpt.cpp:649-677).
    void optimizer_step(float lr, float beta1, float beta2, float decay)
    {
        ++step_;
        const size_t L = c_.layers, D = c_.d_model, F = c_.d_ffn;
        struct Slice { size_t off, n; bool decay; };
        const Slice slices[] = {
            {lay_.wte, size_t(c_.vocab_padded) * D, true}, {lay_.wpe, size_t(c_.max_seq_len) * D, true}, {lay_.ln1_w, L * D, false},
            {lay_.ln1_b, L * D, false}, {lay_.qkv_w, L * D * 3 * D, true}, {lay_.qkv_b, L * 3 * D, false}, {lay_.proj_w, L * D * D, true},
            {lay_.proj_b, L * D, false}, {lay_.ln2_w, L * D, false}, {lay_.ln2_b, L * D, false}, {lay_.up_w, L * D * F, true},
            {lay_.up_b, L * F, false}, {lay_.down_w, L * F * D, true}, {lay_.down_b, L * D, false}, {lay_.lnf_w, D, false}, {lay_.lnf_b, D, false}};
        for (const Slice &s : slices)
            be_->device_adamw_step(bufs_[0] + s.off, bufs_[1] + s.off, bufs_[2] + s.off, bufs_[3] + s.off, static_cast<int>(s.n), lr, beta1, beta2,
                                   1e-8f, s.decay ? decay : 0.0f, step_);
    }

    // the sixteen tensors in packing order: end offset and whether weight decay applies (src/model/gpt.cpp:649-677)
    int segments(long long *ends, unsigned char *decay) const
    {
        const size_t L = c_.layers, D = c_.d_model, F = c_.d_ffn;
        const size_t sizes[16] = {size_t(c_.vocab_padded) * D, size_t(c_.max_seq_len) * D, L * D, L * D, L * D * 3 * D, L * 3 * D, L * D * D, L * D,
                                  L * D, L * D, L * D * F, L * F, L * F * D, L * D, D, D};
        const unsigned char dec[16] = {1, 1, 0, 0, 1, 0, 1, 0, 0, 0, 1, 0, 1, 0, 0, 0};
        long long o = 0;
        for (int t = 0; t < 16; ++t) {
            o += static_cast<long long>(sizes[t]);
            ends[t] = o;
            decay[t] = dec[t];
        }
        return 16;
    }
    float *moment(int which) { return bufs_[2 + which]; }
    bool has_optimizer_state() const { return use_grad_; }
    int step_count() const { return step_; }
    void set_step_count(int s) { step_ = s; }
    int next_step() { return ++step_; }

    float *logits() { return acts_ ? acts_ + a_.logits : nullptr; }
    int batch() const { return B_; }
    int seq() const { return T_; }
    const Config &config() const { return c_; }

private:
    void release_activations()
    {
        if (acts_) be_->device_free(acts_);
        if (agrads_) be_->device_free(agrads_);
        if (gen_) be_->device_free(gen_);
        gen_ = nullptr;
        gen_capacity_ = 0;
        acts_ = agrads_ = nullptr;
        acts_capacity_ = agrads_capacity_ = 0;
    }

    struct ActLayout {
        size_t x_emb, ln1, ln1_mean, ln1_var, qkv, lse, attn, proj, ln2, ln2_mean, ln2_var, up, act, down, lnf, lnf_mean, lnf_var, logits, probs, row_loss, total;
    } a_{};
    struct GradLayout {
        size_t d_ln, d_res, d_x, d_qkv, d_helper, d_f1, d_f2, d_logits, total;
    } g_{};

    IGPTBackend *be_;
    Config c_;
    ParamLayout lay_;
    bool use_grad_;
    float *bufs_[4] = {nullptr, nullptr, nullptr, nullptr};
    float *acts_ = nullptr, *agrads_ = nullptr, *loss_dev_ = nullptr;
    size_t acts_capacity_ = 0, agrads_capacity_ = 0;
    int B_ = 0, T_ = 0, step_ = 0;
    bool defer_embedding_ = false;
    gptb200_ctx *ctx_ = nullptr;   // the backend's context, for the operators that are not part of IGPTBackend
    bool fused_ce_ = false, fused_ce_active_ = false, row_loss_valid_ = false;
    bool fused_gelu_ = false;
    float *gen_ = nullptr;        // KV cache of every layer, then the step's activations, then the device copy of the position
    size_t gen_capacity_ = 0, gen_pos_off_ = 0;
    int gen_batch_ = 0, gen_max_len_ = 0, gen_pos_ = 0;
};

struct ModelHandle {
    B200Backend *backend;
    GptModel *model;
};

}  // namespace

// ---- C entry points (declared in include/gptb200.h) ------------------------------------------------------

struct gptb200_model {
    ModelHandle h;
};

extern "C" {

int gptb200_model_create(gptb200_model **out, const int *cfg, int device, void *stream, int mode, unsigned long seed, int use_grad)
{
    if (!out || !cfg) return GPTB200_ERR_INVALID_ARG;
    for (int i = 0; i < 7; ++i)
        if (cfg[i] <= 0) return GPTB200_ERR_INVALID_ARG;
    Config c{cfg[0], cfg[1], cfg[2], cfg[3], cfg[4], cfg[5], cfg[6]};
    if (c.vocab_padded < c.vocab || c.d_model % c.heads != 0) return GPTB200_ERR_INVALID_ARG;
    // the optimiser-side operators of the interface take the element count as int (backend_interface.h:219-237)
    if (ParamLayout(c).total > size_t(0x7fffffff)) return GPTB200_ERR_TOO_LARGE;
    auto *m = new gptb200_model();
    m->h.backend = new B200Backend(seed, device, stream, mode, /*abort_on_error=*/false);
    m->h.model = m->h.backend->status() == 0 ? new GptModel(m->h.backend, c, use_grad != 0) : nullptr;
    if (m->h.model) m->h.model->set_context(m->h.backend->context());
    const int rc = m->h.backend->status();   // no device, or the parameter buffers could not be allocated
    if (rc != GPTB200_OK) {
        delete m->h.model;
        delete m->h.backend;
        delete m;
        return rc;
    }
    *out = m;
    return GPTB200_OK;
}

int gptb200_model_destroy(gptb200_model *m)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    delete m->h.model;
    delete m->h.backend;
    delete m;
    return GPTB200_OK;
}

gptb200_ctx *gptb200_model_context(gptb200_model *m) { return m ? m->h.backend->context() : nullptr; }
long long gptb200_model_num_params(gptb200_model *m) { return m ? static_cast<long long>(m->h.model->num_params()) : -1; }
float *gptb200_model_weights(gptb200_model *m) { return m ? m->h.model->weights() : nullptr; }
float *gptb200_model_grads(gptb200_model *m) { return m ? m->h.model->grads() : nullptr; }
float *gptb200_model_logits(gptb200_model *m) { return m ? m->h.model->logits() : nullptr; }

// offsets[16] (floats) of wte, wpe, ln_1_w, ln_1_b, qkv_proj_w, qkv_proj_b, attn_proj_w, attn_proj_b, ln_2_w, ln_2_b,
// ffn_up_w, ffn_up_b, ffn_down_w, ffn_down_b, ln_f_w, ln_f_b inside the packed parameter / gradient buffers
int gptb200_model_param_offsets(gptb200_model *m, long long *offsets16)
{
    if (!m || !offsets16) return GPTB200_ERR_INVALID_ARG;
    const ParamLayout &l = m->h.model->layout();
    const size_t v[16] = {l.wte, l.wpe, l.ln1_w, l.ln1_b, l.qkv_w, l.qkv_b, l.proj_w, l.proj_b, l.ln2_w, l.ln2_b, l.up_w, l.up_b, l.down_w, l.down_b,
                          l.lnf_w, l.lnf_b};
    for (int i = 0; i < 16; ++i) offsets16[i] = static_cast<long long>(v[i]);
    return GPTB200_OK;
}

int gptb200_model_init(gptb200_model *m, float mean, float stddev)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->init(mean, stddev);
    return m->h.backend->status();
}

// Raw fp32 parameter image in the reference's checkpoint layout (src/model/gpt.cpp:327-397), from / to host memory.
int gptb200_model_load_weights(gptb200_model *m, const float *host, long long count)
{
    if (!m || !host || count != static_cast<long long>(m->h.model->num_params())) return GPTB200_ERR_INVALID_ARG;
    m->h.backend->device_memcpy_h2d(m->h.model->weights(), host, size_t(count) * sizeof(float));
    return m->h.backend->status();
}

int gptb200_model_read(gptb200_model *m, float *host, long long count, int which)
{
    if (!m || !host || count != static_cast<long long>(m->h.model->num_params()) || which < 0 || which > 1) return GPTB200_ERR_INVALID_ARG;
    m->h.backend->device_memcpy_d2h(host, which == 0 ? m->h.model->weights() : m->h.model->grads(), size_t(count) * sizeof(float));
    return m->h.backend->status();
}

int gptb200_model_load_checkpoint(gptb200_model *m, const char *path)
{
    if (!m || !path) return GPTB200_ERR_INVALID_ARG;
    FILE *fp = fopen(path, "rb");
    if (!fp) return GPTB200_ERR_INVALID_ARG;
    std::vector<float> data(m->h.model->num_params());
    const size_t got = fread(data.data(), sizeof(float), data.size(), fp);
    fclose(fp);
    if (got != data.size()) return GPTB200_ERR_INVALID_ARG;
    return gptb200_model_load_weights(m, data.data(), static_cast<long long>(data.size()));
}

int gptb200_model_save_checkpoint(gptb200_model *m, const char *path)
{
    if (!m || !path) return GPTB200_ERR_INVALID_ARG;
    std::vector<float> data(m->h.model->num_params());
    int rc = gptb200_model_read(m, data.data(), static_cast<long long>(data.size()), 0);
    if (rc) return rc;
    FILE *fp = fopen(path, "wb");
    if (!fp) return GPTB200_ERR_INVALID_ARG;
    const size_t put = fwrite(data.data(), sizeof(float), data.size(), fp);
    fclose(fp);
    return put == data.size() ? GPTB200_OK : GPTB200_ERR_INVALID_ARG;
}

int gptb200_model_set_size(gptb200_model *m, int batch, int seq)
{
    if (!m || batch <= 0 || seq <= 0 || seq > m->h.model->config().max_seq_len) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    if (size_t(batch) * seq * m->h.model->config().vocab_padded > size_t(0x7fffffff)) return GPTB200_ERR_TOO_LARGE;   // the logits tensor is indexed with int
    if (!m->h.model->set_size(batch, seq)) {
        const int rc = m->h.backend->status();
        m->h.backend->clear_status();   // nothing was changed: the model keeps working at its previous size
        return rc;
    }
    return GPTB200_OK;
}

int gptb200_model_zero_grad(gptb200_model *m)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->zero_grad();
    return m->h.backend->status();
}

int gptb200_model_forward(gptb200_model *m, const int *tokens_dev)
{
    if (!m || !tokens_dev || m->h.model->batch() == 0) return GPTB200_ERR_INVALID_ARG;
    m->h.model->forward(tokens_dev);
    return m->h.backend->status();
}

int gptb200_model_backward(gptb200_model *m, const int *tokens_dev, const int *labels_dev, void (*layer_done)(int, void *), void *user)
{
    if (!m || !tokens_dev || !labels_dev || m->h.model->batch() == 0) return GPTB200_ERR_INVALID_ARG;
    m->h.model->backward(tokens_dev, labels_dev, layer_done, user);
    return m->h.backend->status();
}

int gptb200_model_set_fused_cross_entropy(gptb200_model *m, int on)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->set_fused_cross_entropy(on != 0);
    return GPTB200_OK;
}

int gptb200_model_set_fused_gelu_backward(gptb200_model *m, int on)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->set_fused_gelu_backward(on != 0);
    return GPTB200_OK;
}

int gptb200_model_generate_begin(gptb200_model *m, const int *prompt_dev, int batch, int prompt_len, int max_len)
{
    if (!m || !prompt_dev || batch <= 0 || prompt_len <= 0 || max_len < prompt_len || max_len > m->h.model->config().max_seq_len)
        return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    const int rc = m->h.model->generate_begin(m->h.backend->context(), prompt_dev, batch, prompt_len, max_len);
    if (m->h.backend->status() != 0) {
        const int st = m->h.backend->status();
        if (rc == GPTB200_ERR_CUDA) m->h.backend->clear_status();   // an allocation that could not be had: nothing was changed
        return st;
    }
    return rc;
}

int gptb200_model_generate_step(gptb200_model *m, const int *tokens_dev, float *logits_dev)
{
    if (!m || !tokens_dev || !logits_dev) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    const int rc = m->h.model->generate_step(m->h.backend->context(), tokens_dev, logits_dev);
    return rc ? rc : m->h.backend->status();
}

int gptb200_model_generate_position(gptb200_model *m) { return m ? m->h.model->generate_position() : -1; }

int gptb200_model_defer_embedding_backward(gptb200_model *m, int defer)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->set_defer_embedding(defer != 0);
    return GPTB200_OK;
}

float *gptb200_model_embedding_grad(gptb200_model *m) { return m ? m->h.model->embedding_grad() : nullptr; }

int gptb200_model_apply_embedding_grad(gptb200_model *m, const float *rows_dev, const int *tokens_dev, int batch, int seq, float scale)
{
    if (!m || !rows_dev || !tokens_dev || batch <= 0 || seq <= 0 || seq > m->h.model->config().max_seq_len) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    GptModel *g = m->h.model;
    return gptb200_embedding_backward_scaled(m->h.backend->context(), g->grads() + g->wte_offset(), g->grads() + g->wpe_offset(), rows_dev, tokens_dev,
                                             batch, seq, g->config().d_model, scale);
}

int gptb200_model_loss(gptb200_model *m, const int *labels_dev, float *loss_out)
{
    if (!m || !labels_dev || !loss_out) return GPTB200_ERR_INVALID_ARG;
    *loss_out = m->h.model->loss(labels_dev);
    if (m->h.backend->status() != 0) return m->h.backend->status();
    // the copy of the loss has waited for the stream: report a bounded wait that ran out in any kernel of the step
    return gptb200_ctx_synchronize(m->h.backend->context());
}

int gptb200_model_clip(gptb200_model *m, float max_norm, int accum_steps)
{
    if (!m || accum_steps <= 0) return GPTB200_ERR_INVALID_ARG;
    m->h.model->clip(max_norm, accum_steps);
    return m->h.backend->status();
}

int gptb200_model_optimizer_step(gptb200_model *m, float lr, float beta1, float beta2, float weight_decay)
{
    if (!m) return GPTB200_ERR_INVALID_ARG;
    m->h.model->optimizer_step(lr, beta1, beta2, weight_decay);
    return m->h.backend->status();
}

int gptb200_model_clip_and_optimizer_step(gptb200_model *m, float max_norm, int accum_steps, float lr, float beta1, float beta2, float weight_decay)
{
    if (!m || accum_steps <= 0 || !m->h.model->has_optimizer_state()) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    long long ends[16];
    unsigned char decay[16];
    const int n = m->h.model->segments(ends, decay);
    GptModel *g = m->h.model;
    return gptb200_clip_adamw_packed(m->h.backend->context(), g->weights(), g->grads(), g->moment(0), g->moment(1), g->num_params(), ends, decay, n,
                                     max_norm, accum_steps, lr, beta1, beta2, 1e-8f, weight_decay, g->next_step(), nullptr);
}

namespace {

struct StateHeader {          // 64 bytes, little-endian
    char magic[8];            // "GPTB200S"
    int version;              // 1
    int cfg[7];               // max_seq_len, vocab_size, vocab_size_padded, num_layers, num_heads, d_model, d_ffn
    int step;                 // optimiser steps taken
    int has_optimizer;        // 1: the two moment buffers follow the parameters
    long long num_params;
    int reserved[2];
};
static_assert(sizeof(StateHeader) == 64, "header layout");

}  // namespace

int gptb200_model_step_count(gptb200_model *m) { return m ? m->h.model->step_count() : -1; }

int gptb200_model_save_state(gptb200_model *m, const char *path)
{
    if (!m || !path) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    GptModel *g = m->h.model;
    StateHeader h{};
    memcpy(h.magic, "GPTB200S", 8);
    h.version = 1;
    const Config &c = g->config();
    const int cfg[7] = {c.max_seq_len, c.vocab, c.vocab_padded, c.layers, c.heads, c.d_model, c.d_ffn};
    memcpy(h.cfg, cfg, sizeof(cfg));
    h.step = g->step_count();
    h.has_optimizer = g->has_optimizer_state() ? 1 : 0;
    h.num_params = static_cast<long long>(g->num_params());
    FILE *fp = fopen(path, "wb");
    if (!fp) return GPTB200_ERR_INVALID_ARG;
    bool ok = fwrite(&h, sizeof(h), 1, fp) == 1;
    std::vector<float> host(g->num_params());
    float *bufs[3] = {g->weights(), h.has_optimizer ? g->moment(0) : nullptr, h.has_optimizer ? g->moment(1) : nullptr};
    for (float *b : bufs) {
        if (!b || !ok) continue;
        m->h.backend->device_memcpy_d2h(host.data(), b, host.size() * sizeof(float));
        ok = m->h.backend->status() == 0 && fwrite(host.data(), sizeof(float), host.size(), fp) == host.size();
    }
    fclose(fp);
    if (m->h.backend->status() != 0) return m->h.backend->status();
    return ok ? GPTB200_OK : GPTB200_ERR_INVALID_ARG;
}

int gptb200_model_load_state(gptb200_model *m, const char *path)
{
    if (!m || !path) return GPTB200_ERR_INVALID_ARG;
    if (m->h.backend->status() != 0) return m->h.backend->status();
    GptModel *g = m->h.model;
    FILE *fp = fopen(path, "rb");
    if (!fp) return GPTB200_ERR_INVALID_ARG;
    StateHeader h{};
    const Config &c = g->config();
    const int cfg[7] = {c.max_seq_len, c.vocab, c.vocab_padded, c.layers, c.heads, c.d_model, c.d_ffn};
    bool ok = fread(&h, sizeof(h), 1, fp) == 1 && memcmp(h.magic, "GPTB200S", 8) == 0 && h.version == 1 && memcmp(h.cfg, cfg, sizeof(cfg)) == 0 &&
              h.num_params == static_cast<long long>(g->num_params()) && h.step >= 0;
    if (ok) {
        // the whole file is read and checked before anything on the device changes
        const int nbuf = (h.has_optimizer && g->has_optimizer_state()) ? 3 : 1;
        std::vector<std::vector<float>> host(nbuf, std::vector<float>(g->num_params()));
        for (int i = 0; i < nbuf && ok; ++i) ok = fread(host[i].data(), sizeof(float), host[i].size(), fp) == host[i].size();
        if (ok) {
            float *dst[3] = {g->weights(), g->has_optimizer_state() ? g->moment(0) : nullptr, g->has_optimizer_state() ? g->moment(1) : nullptr};
            for (int i = 0; i < nbuf; ++i) m->h.backend->device_memcpy_h2d(dst[i], host[i].data(), host[i].size() * sizeof(float));
            g->set_step_count(nbuf == 3 ? h.step : 0);
        }
    }
    fclose(fp);
    if (m->h.backend->status() != 0) return m->h.backend->status();
    return ok ? GPTB200_OK : GPTB200_ERR_INVALID_ARG;
}

}  // extern "C"
