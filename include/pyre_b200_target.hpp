/* C++ side of the boundary: the reference's speculative-decoding target over the C ABI.
 *
 * Mirrors `spec::Target` (src/spec.rs:106-120 of the reference) as implemented for the Qwen-Next model by `QnTarget`
 * (src/engine_qn.rs:245-253): step -> Model::forward, verify -> Model::forward_multi, keep -> Model::spec_keep,
 * can_verify -> Model::multi_ok, max_window -> Model::spec_max_window, draft -> Model::mtp_draft.  The generation loop that
 * drives a target (spec::generate, src/spec.rs:156-267) and the sampler stay the caller's; this header only gives them the
 * same six calls on a `pb_state`.  Header-only, C++17, no dependency besides pyre_b200.h; errors of the library are thrown as
 * pyre_b200::Error with the library's message.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <limits>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "pyre_b200.h"

namespace pyre_b200 {

struct Error : std::runtime_error {
    int status;
    Error(int s, const std::string& what) : std::runtime_error(what), status(s) {}
};

/* (token, probability) pairs of a draft distribution, as the reference attaches them to sampled drafts */
using Dist = std::vector<std::pair<uint32_t, float>>;
/* one drafted token; `q` is empty for a greedy draft (a point mass) */
struct Draft { uint32_t token; std::optional<Dist> q; };
/* The caller's sampler for drafts (mtp_qsample, src/model/qwen4exp_gguf.rs:3321-3331): given the drafter's logits over the
 * draft vocabulary and the token of every row, returns the drawn token and the distribution it was drawn from. */
using DraftSampler = std::function<std::pair<uint32_t, Dist>(const float* logits, const uint32_t* vocab_ids, int n_ids)>;

class QnTarget {
public:
    /* ctx, model and state stay the caller's (Model and State of the reference: QnTarget borrows both) */
    QnTarget(pb_ctx* ctx, pb_model* model, pb_state* state) : ctx_(ctx), m_(model), st_(state) {
        check(pb_caps_get(m_, &caps_));
        pb_cfg c;
        check(pb_model_cfg(m_, &c));
        vocab_ = c.vocab;
    }

    /* Feed one token, logits of the next position. */
    std::vector<float> step(uint32_t tok) {
        std::vector<float> lg(vocab_);
        check(pb_forward(st_, &tok, 1, lg.data()));
        return lg;
    }
    /* Feed `toks`; logits after each of them. */
    std::vector<std::vector<float>> verify(const std::vector<uint32_t>& toks) {
        const int t = static_cast<int>(toks.size());
        std::vector<float> flat(static_cast<size_t>(t) * vocab_);
        check(pb_verify(st_, toks.data(), t, flat.data()));
        std::vector<std::vector<float>> out(static_cast<size_t>(t));
        for (int j = 0; j < t; j++) out[static_cast<size_t>(j)].assign(flat.begin() + static_cast<std::ptrdiff_t>(j) * vocab_, flat.begin() + static_cast<std::ptrdiff_t>(j + 1) * vocab_);
        return out;
    }
    /* Keep the first `keep` of the last `t` fed tokens. */
    void keep(size_t t, size_t keep) { check(pb_keep(st_, static_cast<int>(t), static_cast<int>(keep))); }
    /* Whether verify + keep are available (else plain decode). */
    bool can_verify() const { return caps_.multi_ok != 0; }
    /* Longest window verify may take while staying identical to plain decode. */
    size_t max_window() const { return caps_.max_window > 0 ? static_cast<size_t>(caps_.max_window) : std::numeric_limits<size_t>::max(); }
    /* Model drafter (MTP): up to k tokens following `history`, whose last token is not fed yet.  nullopt when no drafter is
     * attached (the caller's n-gram drafter takes over, src/spec.rs:207).  With a sampler every token is drawn from the
     * drafter's distribution and carries it. */
    std::optional<std::vector<Draft>> draft(const std::vector<uint32_t>& history, size_t k, float min_p = 0.9f, const DraftSampler* sample = nullptr) {
        if (history.empty()) return std::vector<Draft>{};
        std::vector<uint32_t> ids(k ? k : 1);
        int n = 0;
        Pick pk{sample, {}};
        const int rc = pb_draft_sampled(st_, history.back(), static_cast<int>(k), min_p, sample ? &QnTarget::trampoline : nullptr, &pk, ids.data(), nullptr, &n);
        if (rc == PB_UNSUPPORTED) return std::nullopt;
        check(rc);
        std::vector<Draft> out;
        for (int j = 0; j < n; j++) {
            Draft d{ids[static_cast<size_t>(j)], std::nullopt};
            if (sample && static_cast<size_t>(j) < pk.dists.size()) d.q = std::move(pk.dists[static_cast<size_t>(j)]);
            out.push_back(std::move(d));
        }
        return out;
    }
    /* position of the state = number of tokens fed and kept (State.tokens.len()) */
    int64_t pos() const { int64_t p = 0; check(pb_state_pos(st_, &p)); return p; }

private:
    struct Pick { const DraftSampler* f; std::vector<Dist> dists; };
    static uint32_t trampoline(void* user, const float* logits, const uint32_t* vocab_ids, int n_ids) {
        Pick* p = static_cast<Pick*>(user);
        auto r = (*p->f)(logits, vocab_ids, n_ids);
        p->dists.push_back(std::move(r.second));
        return r.first;
    }
    void check(int rc) const {
        if (rc != 0) throw Error(rc, std::string(pb_last_error(ctx_)));
    }
    pb_ctx* ctx_; pb_model* m_; pb_state* st_;
    pb_caps caps_{};
    int vocab_ = 0;
};

}  // namespace pyre_b200
