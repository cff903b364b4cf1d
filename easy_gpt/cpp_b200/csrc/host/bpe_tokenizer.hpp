// Text <-> token ids for the command line: a byte-level BPE with the reference's rules.
//  * the text is cut at special tokens: the earliest match wins, the longest at the same place
//    (src/tokenizer.cpp:58-75, 270-281);
//  * what lies between is split at whitespace; every word but the first gets one leading space, runs
//    of whitespace and line breaks collapse (src/bpe.cpp:32-62); a word that touches a special token
//    on both sides without whitespace gets no space (src/tokenizer.cpp:85-92);
//  * a word's bytes are mapped to the printable stand-ins of the GPT-2 table (src/bpe.cpp:163-195)
//    and merged pair by pair, lowest merge rank first (src/bpe.cpp:119-161);
//  * tokens that are not in the vocabulary are dropped; BOS is put in front if there is one
//    (src/tokenizer.cpp:129-142).
// All strings are UTF-8.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace easygpt::host {

inline void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += (char)cp;
    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
}

// length in bytes of the UTF-8 sequence that starts with this byte (1 for a stray byte)
inline int utf8_length(unsigned char lead) {
    if (lead < 0x80) return 1;
    if ((lead >> 5) == 0x6) return 2;
    if ((lead >> 4) == 0xE) return 3;
    if ((lead >> 3) == 0x1E) return 4;
    return 1;
}

inline uint32_t utf8_decode(const std::string& s, size_t at, int* length) {
    const unsigned char lead = (unsigned char)s[at];
    int n = utf8_length(lead);
    if (at + n > s.size()) n = 1;
    *length = n;
    if (n == 1) return lead;
    uint32_t cp = lead & (0xFF >> (n + 1));
    for (int i = 1; i < n; ++i) cp = (cp << 6) | ((unsigned char)s[at + i] & 0x3F);
    return cp;
}

// What splits words: the six ASCII white-space characters, as in the reference, which reads words with
// `iss >> word` in the classic locale (src/bpe.cpp:32-62) and asks std::isspace about the bytes beside a
// special token (src/tokenizer.cpp:83-90).  Other Unicode spaces (U+00A0, U+3000, ...) are bytes of a word.
inline bool is_space(uint32_t cp) { return (cp >= 0x09 && cp <= 0x0D) || cp == 0x20; }

class BpeTokenizer {
public:
    BpeTokenizer() {
        // GPT-2's table: printable bytes stand for themselves, the others for the code points from 256 on
        bool keep[256] = {false};
        for (int b = '!'; b <= '~'; ++b) keep[b] = true;
        for (int b = 0xA1; b <= 0xAC; ++b) keep[b] = true;
        for (int b = 0xAE; b <= 0xFF; ++b) keep[b] = true;
        uint32_t extra = 0;
        for (int b = 0; b < 256; ++b) {
            const uint32_t cp = keep[b] ? (uint32_t)b : 256 + extra++;
            append_utf8(byte_to_char_[b], cp);
            char_to_byte_[cp] = (unsigned char)b;
        }
    }

    void add_token(const std::string& token, int32_t id) {
        token_to_id_[token] = id;
        id_to_token_[id] = token;
    }
    // in the order of their ranks (a pair given again takes the later rank)
    void add_merge(const std::string& left, const std::string& right) { rank_[std::make_pair(left, right)] = merges_++; }
    // to be added longest first (ties in the order of the strings)
    void add_special(const std::string& token) { specials_.push_back(token); }
    void set_bos(int32_t id) { bos_ = id; }

    std::vector<std::string> tokenize(const std::string& text) {
        std::vector<std::string> out;
        bool first_word = true, no_space_next = false;
        size_t pos = 0;
        while (pos < text.size()) {
            const std::string* hit = nullptr;
            size_t hit_at = text.size();
            for (const std::string& s : specials_) {                    // longest first; earliest wins
                const size_t at = text.find(s, pos);
                if (at != std::string::npos && at < hit_at) { hit = &s; hit_at = at; }
            }
            if (hit_at > pos && plain(text, pos, hit_at, first_word || no_space_next, out)) first_word = false;
            if (!hit) break;
            out.push_back(*hit);
            const size_t end = hit_at + hit->size();
            no_space_next = hit_at > 0 && !is_space(code_point_before(text, hit_at)) && end < text.size() && !is_space(code_point_at(text, end));
            pos = end;
        }
        return out;
    }

    std::vector<int32_t> encode(const std::string& text) {
        std::vector<int32_t> ids;
        if (bos_ >= 0) ids.push_back(bos_);
        for (const std::string& t : tokenize(text)) {
            auto it = token_to_id_.find(t);
            if (it != token_to_id_.end()) ids.push_back(it->second);    // unknown pieces are dropped
        }
        return ids;
    }

    // bytes of the text (valid UTF-8 only if the ids spell whole characters)
    std::string decode(const int32_t* ids, size_t n) const {
        std::string raw;
        for (size_t i = 0; i < n; ++i) {
            auto it = id_to_token_.find(ids[i]);
            if (it == id_to_token_.end()) continue;
            const std::string& t = it->second;
            for (size_t at = 0; at < t.size();) {
                int len;
                const uint32_t cp = utf8_decode(t, at, &len);
                auto b = char_to_byte_.find(cp);
                if (b != char_to_byte_.end()) raw += (char)b->second;
                else raw.append(t, at, len);                           // a special token's own characters
                at += len;
            }
        }
        return raw;
    }

private:
    static uint32_t code_point_at(const std::string& s, size_t at) {
        int len;
        return utf8_decode(s, at, &len);
    }
    static uint32_t code_point_before(const std::string& s, size_t at) {
        size_t start = at - 1;
        while (start > 0 && ((unsigned char)s[start] & 0xC0) == 0x80) --start;
        return code_point_at(s, start);
    }

    // tokens of text[from, to), which holds no special token; returns whether it held a word
    bool plain(const std::string& text, size_t from, size_t to, bool first_word, std::vector<std::string>& out) {
        bool saw = false;
        size_t at = from;
        while (at < to) {
            int len;
            while (at < to && is_space(utf8_decode(text, at, &len))) at += len;
            const size_t start = at;
            while (at < to && !is_space(utf8_decode(text, at, &len))) at += len;
            if (at > to) at = to;
            if (at == start) break;
            std::string mapped;
            if (!first_word) mapped += byte_to_char_[(unsigned char)' '];
            for (size_t i = start; i < at; ++i) mapped += byte_to_char_[(unsigned char)text[i]];
            first_word = false;
            saw = true;
            const std::vector<std::string>& parts = merge_word(mapped);
            out.insert(out.end(), parts.begin(), parts.end());
        }
        return saw;
    }

    const std::vector<std::string>& merge_word(const std::string& word) {
        auto cached = cache_.find(word);
        if (cached != cache_.end()) return cached->second;
        std::vector<std::string> parts;
        for (size_t at = 0; at < word.size();) {
            const int len = utf8_length((unsigned char)word[at]);
            parts.push_back(word.substr(at, len));
            at += len;
        }
        while (parts.size() > 1) {
            int best = -1;
            size_t where = 0;
            for (size_t i = 0; i + 1 < parts.size(); ++i) {
                auto r = rank_.find(std::make_pair(parts[i], parts[i + 1]));
                if (r != rank_.end() && (best < 0 || r->second < best)) { best = r->second; where = i; }
            }
            if (best < 0) break;
            parts[where] += parts[where + 1];
            parts.erase(parts.begin() + where + 1);
        }
        return cache_.emplace(word, std::move(parts)).first->second;
    }

    std::string byte_to_char_[256];
    std::unordered_map<uint32_t, unsigned char> char_to_byte_;
    std::unordered_map<std::string, int32_t> token_to_id_;
    std::unordered_map<int32_t, std::string> id_to_token_;
    std::map<std::pair<std::string, std::string>, int> rank_;
    std::vector<std::string> specials_;
    std::unordered_map<std::string, std::vector<std::string>> cache_;
    int32_t bos_ = -1;
    int merges_ = 0;
};

}  // namespace easygpt::host
