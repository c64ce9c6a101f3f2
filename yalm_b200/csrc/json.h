// A small JSON document reader for model configuration files (config.json of a checkpoint directory): objects, arrays,
// strings, numbers, true / false / null.  The safetensors header keeps its own streaming reader in codec.cpp; this
// one builds a tree, because a layered model's configuration nests (a list of layers, each with a mixer and a
// feed-forward description).
#pragma once

#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace yalm {

struct JValue {
	enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
	bool b = false;
	double num = 0.0;
	std::string str;
	std::vector<JValue> arr;
	std::vector<std::pair<std::string, JValue>> obj; // in file order

	bool is_null() const { return kind == Null; }
	bool is_object() const { return kind == Object; }
	bool is_array() const { return kind == Array; }
	// member lookup; a static null value when absent or when this is not an object
	const JValue &operator[](const char *key) const {
		static const JValue none;
		if (kind != Object) return none;
		for (const auto &kv : obj)
			if (kv.first == key) return kv.second;
		return none;
	}
	bool has(const char *key) const { return !(*this)[key].is_null(); }
	double number(double dflt) const { return kind == Number ? num : kind == Bool ? (b ? 1.0 : 0.0) : dflt; }
	int integer(int dflt) const { return kind == Number ? (int)num : kind == Bool ? (int)b : dflt; }
	bool truthy() const { return kind == Bool ? b : kind == Number ? num != 0.0 : kind == String ? !str.empty() : kind != Null; }
	const std::string &string_or(const std::string &dflt) const { return kind == String ? str : dflt; }
};

// Parses `text`; returns false (and leaves *out undefined) on malformed input.
bool json_parse(const char *text, size_t size, JValue *out);

} // namespace yalm
