// Model registry and the configuration readers of the layered architectures (arch.h), plus the JSON tree reader.
#include "arch.h"

#include "yalm_api.h"

#include <algorithm>
#include <cstring>

namespace yalm {

// ---- JSON ------------------------------------------------------------------------------------------------------------
namespace {
struct JCursor {
	const char *p, *end;
	int depth = 0;
	void ws() {
		while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
	}
	bool lit(const char *s) {
		const size_t n = strlen(s);
		if ((size_t)(end - p) >= n && memcmp(p, s, n) == 0) {
			p += n;
			return true;
		}
		return false;
	}
	bool string(std::string *out) {
		if (p >= end || *p != '"') return false;
		++p;
		while (p < end && *p != '"') {
			if (*p == '\\' && p + 1 < end) {
				++p;
				switch (*p) {
				case 'n': *out += '\n'; break;
				case 't': *out += '\t'; break;
				case 'r': *out += '\r'; break;
				case 'b': *out += '\b'; break;
				case 'f': *out += '\f'; break;
				case 'u': {
					if (p + 4 >= end) return false;
					const unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
					p += 4;
					if (cp < 0x80) *out += (char)cp;
					else if (cp < 0x800) *out += (char)(0xC0 | (cp >> 6)), *out += (char)(0x80 | (cp & 0x3F));
					else *out += (char)(0xE0 | (cp >> 12)), *out += (char)(0x80 | ((cp >> 6) & 0x3F)), *out += (char)(0x80 | (cp & 0x3F));
					break;
				}
				default: *out += *p;
				}
				++p;
			} else {
				*out += *p++;
			}
		}
		if (p >= end) return false;
		++p;
		return true;
	}
	bool value(JValue *v) {
		if (++depth > 64) return false;
		ws();
		if (p >= end) return false;
		bool ok = true;
		if (*p == '{') {
			++p;
			v->kind = JValue::Object;
			ws();
			if (p < end && *p == '}') ++p;
			else {
				for (;;) {
					ws();
					std::string key;
					if (!string(&key)) return false;
					ws();
					if (p >= end || *p++ != ':') return false;
					v->obj.emplace_back(key, JValue());
					if (!value(&v->obj.back().second)) return false;
					ws();
					if (p < end && *p == ',') { ++p; continue; }
					if (p < end && *p == '}') { ++p; break; }
					return false;
				}
			}
		} else if (*p == '[') {
			++p;
			v->kind = JValue::Array;
			ws();
			if (p < end && *p == ']') ++p;
			else {
				for (;;) {
					v->arr.emplace_back();
					if (!value(&v->arr.back())) return false;
					ws();
					if (p < end && *p == ',') { ++p; continue; }
					if (p < end && *p == ']') { ++p; break; }
					return false;
				}
			}
		} else if (*p == '"') {
			v->kind = JValue::String;
			ok = string(&v->str);
		} else if (lit("true")) {
			v->kind = JValue::Bool, v->b = true;
		} else if (lit("false")) {
			v->kind = JValue::Bool, v->b = false;
		} else if (lit("null")) {
			v->kind = JValue::Null;
		} else {
			// strtod needs a terminated buffer: numbers are short, copy the candidate characters
			char buf[64];
			size_t n = 0;
			while (p + n < end && n < sizeof(buf) - 1 && strchr("+-0123456789.eE", p[n])) ++n;
			if (n == 0) return false;
			memcpy(buf, p, n);
			buf[n] = 0;
			char *e = nullptr;
			v->num = strtod(buf, &e);
			if (e == buf) return false;
			p += e - buf;
			v->kind = JValue::Number;
		}
		--depth;
		return ok;
	}
};
} // namespace

bool json_parse(const char *text, size_t size, JValue *out) {
	JCursor c{text, text + size};
	*out = JValue();
	if (!c.value(out)) return false;
	c.ws();
	return c.p == c.end;
}

// ---- StackSpec -------------------------------------------------------------------------------------------------------
int StackSpec::max_q_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.heads * l.mix.dim);
	return m;
}
int StackSpec::max_kv_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.kv_heads * l.mix.dim);
	return m;
}
int StackSpec::max_v_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.kv_heads * l.mix.vdim);
	return m;
}
int StackSpec::max_o_dim() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.mix.heads * l.mix.vdim);
	return m;
}
int StackSpec::max_ff() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.ffn.ff);
	return m;
}
int StackSpec::max_top() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.ffn.top);
	return m;
}
int StackSpec::max_experts() const {
	int m = 0;
	for (const LayerSpec &l : layers) m = std::max(m, l.ffn.experts);
	return m;
}

// ---- Retezen ---------------------------------------------------------------------------------------------------------
// A decoder-only stack: learned absolute positions; every sublayer reads the residual stream itself and its OUTPUT is
// RMS-normalised (weights stored around zero) before it is added back; attention without rotation, with an RMS norm over
// the whole q and k projections, a sliding window plus one mean key/value per block of tokens that has left the window,
// and values blended with the first blending layer's; feed-forward either dense (gate clamped from above, up clamped
// both ways, g * sigmoid(1.702 g) * (u + 1)) or a mixture of SiLU-gated experts routed by sigmoid scores that scale the
// expert's input.
namespace {

std::string retezen_tensor(int layer, TensorRole role, int expert) {
	const std::string l = "l" + std::to_string(layer) + ".";
	const std::string e = expert >= 0 ? "e" + std::to_string(expert) + "." : "";
	switch (role) {
	case TensorRole::Embed: return "embed";
	case TensorRole::Positions: return "pos";
	case TensorRole::FinalNorm: return "final.norm";
	case TensorRole::Head: return "head";
	case TensorRole::Norm1: return l + "norm1";
	case TensorRole::Norm2: return l + "norm2";
	case TensorRole::Wq: return l + "mix.q";
	case TensorRole::Wk: return l + "mix.k";
	case TensorRole::Wv: return l + "mix.v";
	case TensorRole::Wo: return l + "mix.o";
	case TensorRole::QNorm: return l + "mix.q.norm";
	case TensorRole::KNorm: return l + "mix.k.norm";
	case TensorRole::VMix: return l + "mix.vmix";
	case TensorRole::Gate: return l + "mlp." + e + "gate";
	case TensorRole::Up: return l + "mlp." + e + "up";
	case TensorRole::Down: return l + "mlp." + e + "down";
	case TensorRole::Router: return l + "mlp.router";
	}
	return "";
}

int fail(const char *what) {
	fprintf(stderr, "yalm_b200: Retezen config.json: %s\n", what);
	return YALM_EFORMAT;
}

int configure_retezen(const JValue &j, Config &cfg) {
	auto spec = std::make_shared<StackSpec>();
	StackSpec &s = *spec;
	s.arch = "Retezen";
	s.width = j["width"].integer(0);
	s.vocab = j["vocab"].integer(0);
	s.max_positions = j["max_positions"].integer(0);
	s.norm_eps = (float)j["norm"]["eps"].number(1e-5);
	s.logit_scale = (float)j["logit_scale"].number(1.0);
	s.norm_one_plus = true;
	s.norm_on_output = true;
	s.learned_positions = true;
	s.tensor_name = retezen_tensor;
	if (s.width < 1 || s.vocab < 1 || s.max_positions < 1) return fail("width, vocab and max_positions must be positive");
	const JValue &layers = j["layers"];
	if (!layers.is_array() || layers.arr.empty()) return fail("'layers' must be a non-empty list");
	for (const JValue &jl : layers.arr) {
		LayerSpec L;
		if (jl["type"].string_or("") != "attention") return fail("unknown layer type (this build has: attention)");
		const JValue &m = jl["mixer"];
		L.mix.heads = m["heads"].integer(0);
		L.mix.kv_heads = m["kv_heads"].integer(L.mix.heads);
		L.mix.dim = m["dim"].integer(0);
		L.mix.vdim = m["vdim"].integer(L.mix.dim);
		L.mix.scale = (float)m["scale"].number(1.0);
		L.mix.window = m["mask"]["size"].integer(0);
		L.mix.pool = m["mask"]["pool"].integer(0);
		L.mix.qk_norm = QkNorm::WholeProjection;
		L.mix.v_mix = m["v_mix"].truthy();
		if (L.mix.heads < 1 || L.mix.kv_heads < 1 || L.mix.heads % L.mix.kv_heads || L.mix.dim < 1 || L.mix.vdim < 1 || L.mix.window < 0 ||
		    L.mix.pool < 0)
			return fail("bad mixer sizes");
		if (L.mix.window == 0) L.mix.pool = 0; // nothing ever leaves an unbounded window
		const JValue &f = jl["mlp"];
		if (f.is_object()) {
			const std::string kind = f["kind"].string_or("");
			if (kind == "dense") {
				L.ffn.kind = FfnSpec::Dense;
				L.ffn.ff = f["ff"].integer(0);
				L.ffn.act = GluAct::SigmoidScaled;
				L.ffn.act_alpha = 1.702f;
				L.ffn.limit = (float)f["limit"].number(0.0);
				L.ffn.up_offset = 1.f;
			} else if (kind == "moe") {
				L.ffn.kind = FfnSpec::Moe;
				L.ffn.ff = f["expert"]["ff"].integer(0);
				L.ffn.act = GluAct::Silu;
				L.ffn.experts = f["router"]["experts"].integer(0);
				L.ffn.top = f["router"]["top"].integer(0);
				L.ffn.score = RouterScore::Sigmoid;
				L.ffn.renormalize = false;
				L.ffn.weight_on_input = true;
				if (L.ffn.experts < 1 || L.ffn.top < 1 || L.ffn.top > L.ffn.experts) return fail("bad router sizes");
			} else
				return fail("unknown mlp kind (this build has: dense, moe)");
			if (L.ffn.ff < 1) return fail("bad feed-forward size");
		}
		s.layers.push_back(L);
	}
	// summary fields the rest of the library sizes scratch buffers and reports from
	cfg.stack = spec;
	cfg.dim = s.width;
	cfg.vocab_size = s.vocab;
	cfg.n_layers = (int)s.layers.size();
	cfg.max_seq_len = s.max_positions;
	cfg.norm_eps = s.norm_eps;
	cfg.hidden_dim = std::max(1, s.max_ff());
	cfg.n_heads = s.layers[0].mix.heads, cfg.n_kv_heads = s.layers[0].mix.kv_heads;
	cfg.head_dim = std::max(s.layers[0].mix.dim, s.layers[0].mix.vdim);
	for (const LayerSpec &l : s.layers) // scratch sizing: heads * head_dim covers every layer's q and attention output
		while (cfg.n_heads * cfg.head_dim < std::max(l.mix.heads * l.mix.dim, l.mix.heads * l.mix.vdim)) cfg.head_dim *= 2;
	cfg.rotary_dim = 0;
	cfg.n_experts = s.max_experts(), cfg.n_experts_active = s.max_top();
	return 0;
}

const ArchEntry kArchs[] = {
    {"Retezen", configure_retezen},
};

} // namespace

const ArchEntry *find_arch(const std::string &name) {
	for (const ArchEntry &a : kArchs)
		if (name == a.name) return &a;
	return nullptr;
}

std::string arch_names() {
	std::string out;
	for (const ArchEntry &a : kArchs) out += (out.empty() ? "" : ", ") + std::string(a.name);
	return out;
}

} // namespace yalm
