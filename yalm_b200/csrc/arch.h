// Model registry.  A checkpoint names its architecture (a `.yalm` file implicitly: the reference's Llama / Mistral /
// Mixtral block, src/model.cpp:17-75; a checkpoint directory through "architecture" in its config.json) and the
// registry turns the configuration into what Model needs: either the homogeneous Config fields the reference has, or
// a StackSpec — a list of layers, each with its own token mixer and feed-forward description and its own sizes.  The
// layered executor (stack.cpp) knows mechanisms and their parameters, not model names: a new design registers a
// reader that fills a StackSpec from its configuration and names its tensors.
#pragma once

#include "json.h"

#include <string>
#include <vector>

struct Config;

namespace yalm {

// Normalisation of q and k before the scores.
enum class QkNorm { None, WholeProjection /* RMS over all heads' channels at once, one weight per channel */ };
// Gated feed-forward activations: y = act(g) * (u + up_offset), with optional clamps on g (from above) and u (both sides).
enum class GluAct { Silu, Gelu, SigmoidScaled /* g * sigmoid(alpha * g) */ };
// How router logits become expert scores.
enum class RouterScore { Softmax, Sigmoid };

struct MixerSpec {
	int heads = 0, kv_heads = 0; // query head h reads key/value head h / (heads / kv_heads)
	int dim = 0, vdim = 0;       // per-head query/key size and value size
	float scale = 1.f;           // score = (q . k) * scale
	int window = 0;              // query i sees keys j with 0 <= i - j < window; 0: all earlier keys
	int pool = 0;                // > 0: beside the window, one mean key/value per block of `pool` tokens lying wholly before it
	QkNorm qk_norm = QkNorm::None;
	bool v_mix = false;          // values blended with the first v_mix layer's values of the same token
};

struct FfnSpec {
	enum Kind { None, Dense, Moe } kind = None;
	int ff = 0;                  // hidden size (per expert for Moe)
	GluAct act = GluAct::Silu;
	float act_alpha = 1.f;       // SigmoidScaled only
	float limit = 0.f;           // > 0: g = min(g, limit), u = clamp(u, -limit, limit)
	float up_offset = 0.f;
	int experts = 0, top = 0;
	RouterScore score = RouterScore::Softmax;
	bool renormalize = false;    // selected scores divided by their sum
	bool weight_on_input = false; // expert(w * h) instead of w * expert(h)
};

struct LayerSpec {
	MixerSpec mix;
	FfnSpec ffn;
};

enum class TensorRole { Embed, Positions, FinalNorm, Head, Norm1, Norm2, Wq, Wk, Wv, Wo, QNorm, KNorm, VMix, Gate, Up, Down, Router };

struct StackSpec {
	std::string arch;
	std::vector<LayerSpec> layers;
	int width = 0, vocab = 0, max_positions = 0;
	float norm_eps = 1e-5f;
	bool norm_one_plus = false;    // norm weights stored around zero: x / rms * (1 + w)
	bool norm_on_output = false;   // x += norm(sublayer(x)) with the sublayer reading x itself, instead of x += sublayer(norm(x))
	bool learned_positions = false; // x = embed[token] + positions[p]
	float logit_scale = 1.f;
	// name of a tensor in the checkpoint; `expert` < 0 for tensors that are not per expert
	std::string (*tensor_name)(int layer, TensorRole role, int expert) = nullptr;

	int max_q_dim() const;  // max over layers of heads * dim
	int max_kv_dim() const; // kv_heads * dim
	int max_v_dim() const;  // kv_heads * vdim
	int max_o_dim() const;  // heads * vdim
	int max_ff() const;
	int max_top() const;
	int max_experts() const;
};

struct ArchEntry {
	const char *name;
	// Fills cfg (Config::stack and the summary fields) from a parsed config.json; returns 0 or YALM_EFORMAT.
	int (*configure)(const JValue &json, Config &cfg);
};

const ArchEntry *find_arch(const std::string &name);
// All registered names, for messages.
std::string arch_names();

} // namespace yalm
