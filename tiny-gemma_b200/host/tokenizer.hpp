// sentencepiece::Tokenizer with the interface and the results of the reference's
// csrc/include/tokenizer.hpp (constructor :77-111, encode :113-199, decode :201-233), written from
// its behaviour. It reads the tokenizer file the reference's py/convert.py:108-113 writes:
//
//   uint32 max_token_length, then per vocabulary entry: float score, uint32 nbytes, nbytes of UTF-8
//   ("▁" already replaced by a space, ids bos/eos renamed "<bos>" / "<eos>").
//
// encode: <bos> [+ chat prefix <start_of_turn> user \n], one token per UTF-8 code point (at most four
// bytes; an unknown code point falls back to its bytes, token id = byte + 3), then repeated merging of the
// adjacent pair whose concatenation is a vocabulary entry with the highest score (the first such pair on
// equal scores) until no pair merges, [+ chat suffix <end_of_turn> \n <start_of_turn> model \n].
//
// Behaviour kept on purpose, because callers compare outputs with the reference:
//   * the merge pass runs over the whole list, <bos> and the chat prefix included;
//   * a leading space is stripped only after token id 1 (prev_token == 1);
//   * texts are found by binary search (equality first, midpoint (lo + hi) / 2) in the vocabulary sorted with
//     std::sort on the text alone, so of several entries with the same text (" " and the former "▁" can
//     collide) the same one is found as by the reference built with the same standard library.
// One deliberate difference: a byte token "<0xNN>" decodes to the byte NN. The reference's decode throws
// std::invalid_argument there (it hands "xNN" to std::stoi), so no output of it can differ. A "<0xNNN>"
// piece above 0xFF is left as it is.
#pragma once
#include <algorithm>
#include <cstdint>
#include <fstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace sentencepiece {

class Tokenizer {
	int bos_id_, eos_id_, vocab_size_;
	unsigned max_token_length_ = 0;
	bool chat_format_;
	// https://ai.google.dev/gemma/docs/core/prompt-structure (the ids of the Gemma-3 vocabulary)
	static constexpr int sot_id = 105, eot_id = 106, newline_id = 107, user_id = 2364, model_id = 4368;
	std::vector<std::string> vocab_;
	std::vector<float> scores_;
	struct Entry {
		std::string_view text;  // view into vocab_ (never resized after construction)
		int id;
	};
	std::vector<Entry> sorted_;

	int lookup(std::string_view s) const {
		int lo = 0, hi = vocab_size_ - 1;
		while (lo <= hi) {
			const int mid = (lo + hi) / 2;
			const std::string_view &m = sorted_[mid].text;
			if (m == s) return sorted_[mid].id;
			if (m > s)
				hi = mid - 1;
			else
				lo = mid + 1;
		}
		return -1;
	}
	static bool is_continuation(char c) { return (static_cast<uint8_t>(c) & 0xC0) == 0x80; }
	static int hex_digit(char c) {
		if (c >= '0' && c <= '9') return c - '0';
		if (c >= 'a' && c <= 'f') return c - 'a' + 10;
		if (c >= 'A' && c <= 'F') return c - 'A' + 10;
		return -1;
	}
	// "<0x" + 2 or 3 hex digits + ">" -> value, else -1
	static int byte_piece_value(const std::string &p) {
		if (p.size() < 6 || p.size() > 7 || p[0] != '<' || p[1] != '0' || p[2] != 'x' || p.back() != '>') return -1;
		int v = 0;
		for (size_t i = 3; i + 1 < p.size(); i++) {
			const int d = hex_digit(p[i]);
			if (d < 0) return -1;
			v = v * 16 + d;
		}
		return v;
	}

   public:
	Tokenizer(const std::string &model_path, const int bos_id, const int eos_id, const int vocab_size, bool chat_format)
	    : bos_id_(bos_id), eos_id_(eos_id), vocab_size_(vocab_size), chat_format_(chat_format) {
		std::ifstream f(model_path, std::ios::binary);
		if (!f) throw std::runtime_error("Cannot open model file: " + model_path);
		uint32_t max_len = 0;
		f.read(reinterpret_cast<char *>(&max_len), sizeof max_len);
		max_token_length_ = max_len;
		vocab_.resize(vocab_size);
		scores_.resize(vocab_size);
		for (int i = 0; i < vocab_size; i++) {
			float score = 0.0f;
			uint32_t nbytes = 0;
			f.read(reinterpret_cast<char *>(&score), sizeof score);
			f.read(reinterpret_cast<char *>(&nbytes), sizeof nbytes);
			if (!f) throw std::runtime_error("Tokenizer file ends before entry " + std::to_string(i) + ": " + model_path);
			vocab_[i].assign(nbytes, '\0');
			f.read(vocab_[i].data(), nbytes);
			scores_[i] = score;
		}
		sorted_.reserve(vocab_size);
		for (int i = 0; i < vocab_size; i++) sorted_.push_back({std::string_view(vocab_[i]), i});
		std::sort(sorted_.begin(), sorted_.end(), [](const Entry &a, const Entry &b) { return a.text < b.text; });
	}
	Tokenizer(const Tokenizer &) = delete;
	Tokenizer &operator=(const Tokenizer &) = delete;

	std::vector<int> encode(const std::string &text) {
		std::vector<int> tokens{bos_id_};
		if (chat_format_) tokens.insert(tokens.end(), {sot_id, user_id, newline_id});
		// one token per code point: a lead byte opens a piece, continuation bytes extend it; the piece is
		// looked up when the next byte is not a continuation or the piece has four bytes (so in malformed
		// text a fifth continuation byte extends the same piece and is looked up again with it)
		std::string piece;
		for (size_t i = 0; i < text.size(); i++) {
			if (!is_continuation(text[i])) piece.clear();
			piece.push_back(text[i]);
			if (i + 1 < text.size() && is_continuation(text[i + 1]) && piece.size() < 4) continue;
			const int id = lookup(piece);
			if (id >= 0) {
				tokens.push_back(id);
			} else {
				for (char c : piece) tokens.push_back(int(static_cast<uint8_t>(c)) + 3);  // after <unk>, <s>, </s>
			}
		}
		// merges, best score first; strict > keeps the leftmost pair among equal scores
		std::string merged;
		for (;;) {
			float best_score = -1e10f;
			int best_id = -1;
			size_t best_at = 0;
			for (size_t i = 0; i + 1 < tokens.size(); i++) {
				merged.assign(vocab_[tokens[i]]);
				merged.append(vocab_[tokens[i + 1]]);
				const int id = lookup(merged);
				if (id >= 0 && scores_[id] > best_score) {
					best_score = scores_[id];
					best_id = id;
					best_at = i;
				}
			}
			if (best_id < 0) break;
			tokens[best_at] = best_id;
			tokens.erase(tokens.begin() + long(best_at) + 1);
		}
		if (chat_format_) tokens.insert(tokens.end(), {eot_id, newline_id, sot_id, model_id, newline_id});
		return tokens;
	}

	std::string decode(int token, int prev_token) {
		std::string piece = vocab_[token];
		if (prev_token == 1 && !piece.empty() && piece[0] == ' ') piece.erase(0, 1);
		const int v = byte_piece_value(piece);
		if (v >= 0 && v < 256) piece.assign(1, char(v));
		return piece;
	}

	std::string decode(const std::vector<int> &tokens) {
		std::string out = decode(bos_id_, -1);
		int prev = bos_id_;
		for (int t : tokens) {
			if (t != bos_id_ && t != eos_id_) out += decode(t, prev);
			prev = t;
		}
		return out;
	}

	int get_bos_id() const { return bos_id_; }
	int get_eos_id() const { return eos_id_; }
	int get_eot_id() const { return eot_id; }
	int get_vocab_size() const { return vocab_size_; }
};

}  // namespace sentencepiece
