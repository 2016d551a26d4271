// Grammar-constrained decoding on the host: a byte-level JSON recogniser driven token by token, and the token mask
// it induces over a vocabulary.  For every step the sampler asks which tokens keep the output a prefix of a valid
// JSON document; the engine masks the others to -inf before arg-max / sampling, then feeds the chosen token back.
//
// Counterpart of the reference's JSON grammar mode (zig/pkg/inference/src/pipelines/grammar.zig: a token byte table
// plus a state machine stepped per candidate token).  The recogniser is a deterministic pushdown automaton:
// a stack of open containers (object / array, depth-limited) and a mode that says what may come next.  It is
// strict RFC 8259 JSON (no trailing commas, no leading zeros, escapes checked, control bytes rejected inside
// strings); bytes >= 0x80 inside strings are accepted as UTF-8 payload without validating the sequence.
#include <stdint.h>
#include <string.h>

#include <vector>

namespace {

enum Mode : uint8_t {
  kValue,            // a value must start here
  kObjFirst,         // after '{': a key string or '}'
  kObjKey,           // after ',' in an object: a key string
  kObjColon,         // after a key: ':'
  kObjNext,          // after a member value: ',' or '}'
  kArrFirst,         // after '[': a value or ']'
  kArrNext,          // after an element: ',' or ']'
  kString, kStringEsc, kStringU1, kStringU2, kStringU3, kStringU4,
  kNumMinus, kNumZero, kNumInt, kNumDot, kNumFrac, kNumE, kNumESign, kNumExp,
  kLiteral,          // inside true / false / null
  kDone,             // a complete top-level value has been read; only whitespace may follow
};

constexpr int kMaxDepth = 64;

struct JsonState {
  uint8_t mode = kValue;
  uint8_t depth = 0;
  uint8_t string_is_key = 0;
  uint8_t lit_id = 0, lit_pos = 0;
  uint8_t root_object_only = 0;
  char stack[kMaxDepth];  // 'O' or 'A'
};

const char* const kLiterals[3] = {"true", "false", "null"};

inline bool is_ws(uint8_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r'; }
inline bool is_digit(uint8_t c) { return c >= '0' && c <= '9'; }
inline bool is_hex(uint8_t c) { return is_digit(c) || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F'); }

inline void value_done(JsonState& s) {
  if (s.depth == 0) s.mode = kDone;
  else s.mode = s.stack[s.depth - 1] == 'O' ? kObjNext : kArrNext;
}

bool start_value(JsonState& s, uint8_t c) {
  if (s.depth == 0 && s.root_object_only && c != '{') return false;
  switch (c) {
    case '{':
      if (s.depth >= kMaxDepth) return false;
      s.stack[s.depth++] = 'O'; s.mode = kObjFirst; return true;
    case '[':
      if (s.depth >= kMaxDepth) return false;
      s.stack[s.depth++] = 'A'; s.mode = kArrFirst; return true;
    case '"': s.mode = kString; s.string_is_key = 0; return true;
    case '-': s.mode = kNumMinus; return true;
    case '0': s.mode = kNumZero; return true;
    case 't': s.mode = kLiteral; s.lit_id = 0; s.lit_pos = 1; return true;
    case 'f': s.mode = kLiteral; s.lit_id = 1; s.lit_pos = 1; return true;
    case 'n': s.mode = kLiteral; s.lit_id = 2; s.lit_pos = 1; return true;
    default:
      if (c >= '1' && c <= '9') { s.mode = kNumInt; return true; }
      return false;
  }
}

// Consumes one byte; false = the byte cannot follow (state is then unspecified: callers step a copy).
bool step(JsonState& s, uint8_t c) {
  for (;;) {
    switch (s.mode) {
      case kValue:
        if (is_ws(c)) return true;
        return start_value(s, c);
      case kObjFirst:
        if (is_ws(c)) return true;
        if (c == '}') { --s.depth; value_done(s); return true; }
        if (c == '"') { s.mode = kString; s.string_is_key = 1; return true; }
        return false;
      case kObjKey:
        if (is_ws(c)) return true;
        if (c == '"') { s.mode = kString; s.string_is_key = 1; return true; }
        return false;
      case kObjColon:
        if (is_ws(c)) return true;
        if (c == ':') { s.mode = kValue; return true; }
        return false;
      case kObjNext:
        if (is_ws(c)) return true;
        if (c == ',') { s.mode = kObjKey; return true; }
        if (c == '}') { --s.depth; value_done(s); return true; }
        return false;
      case kArrFirst:
        if (is_ws(c)) return true;
        if (c == ']') { --s.depth; value_done(s); return true; }
        return start_value(s, c);
      case kArrNext:
        if (is_ws(c)) return true;
        if (c == ',') { s.mode = kValue; return true; }
        if (c == ']') { --s.depth; value_done(s); return true; }
        return false;
      case kString:
        if (c == '"') {
          if (s.string_is_key) s.mode = kObjColon; else value_done(s);
          return true;
        }
        if (c == '\\') { s.mode = kStringEsc; return true; }
        return c >= 0x20;
      case kStringEsc:
        if (c == 'u') { s.mode = kStringU1; return true; }
        if (c == '"' || c == '\\' || c == '/' || c == 'b' || c == 'f' || c == 'n' || c == 'r' || c == 't') {
          s.mode = kString; return true;
        }
        return false;
      case kStringU1: case kStringU2: case kStringU3:
        if (!is_hex(c)) return false;
        ++s.mode; return true;
      case kStringU4:
        if (!is_hex(c)) return false;
        s.mode = kString; return true;
      case kNumMinus:
        if (c == '0') { s.mode = kNumZero; return true; }
        if (c >= '1' && c <= '9') { s.mode = kNumInt; return true; }
        return false;
      case kNumZero:
        if (c == '.') { s.mode = kNumDot; return true; }
        if (c == 'e' || c == 'E') { s.mode = kNumE; return true; }
        if (is_digit(c)) return false;  // no leading zeros
        value_done(s); continue;         // the number ended: re-read this byte as what follows a value
      case kNumInt:
        if (is_digit(c)) return true;
        if (c == '.') { s.mode = kNumDot; return true; }
        if (c == 'e' || c == 'E') { s.mode = kNumE; return true; }
        value_done(s); continue;
      case kNumDot:
        if (is_digit(c)) { s.mode = kNumFrac; return true; }
        return false;
      case kNumFrac:
        if (is_digit(c)) return true;
        if (c == 'e' || c == 'E') { s.mode = kNumE; return true; }
        value_done(s); continue;
      case kNumE:
        if (c == '+' || c == '-') { s.mode = kNumESign; return true; }
        if (is_digit(c)) { s.mode = kNumExp; return true; }
        return false;
      case kNumESign:
        if (is_digit(c)) { s.mode = kNumExp; return true; }
        return false;
      case kNumExp:
        if (is_digit(c)) return true;
        value_done(s); continue;
      case kLiteral: {
        const char* lit = kLiterals[s.lit_id];
        if (static_cast<uint8_t>(lit[s.lit_pos]) != c) return false;
        if (lit[++s.lit_pos] == 0) value_done(s);
        return true;
      }
      case kDone:
        return is_ws(c);
      default:
        return false;
    }
  }
}

bool complete(const JsonState& s) {
  if (s.mode == kDone) return true;
  // a top-level number has no closing delimiter: it is complete as soon as it could end
  return s.depth == 0 && (s.mode == kNumZero || s.mode == kNumInt || s.mode == kNumFrac || s.mode == kNumExp);
}

struct Grammar {
  JsonState state;
  std::vector<uint8_t> bytes;      // concatenated token byte strings
  std::vector<int64_t> offsets;    // n_tokens + 1
};

}  // namespace

extern "C" {

void* afb_grammar_json_new(int root_object_only) {
  Grammar* g = new Grammar();
  g->state.root_object_only = root_object_only ? 1 : 0;
  return g;
}

void afb_grammar_free(void* h) { delete static_cast<Grammar*>(h); }

void afb_grammar_reset(void* h) {
  Grammar* g = static_cast<Grammar*>(h);
  const uint8_t roo = g->state.root_object_only;
  g->state = JsonState();
  g->state.root_object_only = roo;
}

// Token byte table: token t is bytes[offsets[t] .. offsets[t + 1]).  Empty tokens (special tokens) are never allowed.
int afb_grammar_set_vocab(void* h, const uint8_t* bytes, const int64_t* offsets, int n_tokens) {
  Grammar* g = static_cast<Grammar*>(h);
  if (n_tokens < 0) return -1;
  g->offsets.assign(offsets, offsets + n_tokens + 1);
  g->bytes.assign(bytes, bytes + offsets[n_tokens]);
  return 0;
}

// allowed[t] = 1 if appending token t keeps the output a valid JSON prefix.  Returns the number allowed.
int afb_grammar_mask(void* h, uint8_t* allowed) {
  Grammar* g = static_cast<Grammar*>(h);
  const int n = static_cast<int>(g->offsets.size()) - 1;
  int count = 0;
  for (int t = 0; t < n; ++t) {
    const int64_t b = g->offsets[t], e = g->offsets[t + 1];
    bool ok = e > b;
    if (ok) {
      JsonState s = g->state;
      for (int64_t i = b; i < e; ++i) {
        if (!step(s, g->bytes[i])) { ok = false; break; }
      }
    }
    allowed[t] = ok ? 1 : 0;
    count += ok ? 1 : 0;
  }
  return count;
}

// Advances by raw bytes; returns 1 if all were accepted (state advanced), 0 if not (state unchanged).
int afb_grammar_accept_bytes(void* h, const uint8_t* bytes, int n) {
  Grammar* g = static_cast<Grammar*>(h);
  JsonState s = g->state;
  for (int i = 0; i < n; ++i)
    if (!step(s, bytes[i])) return 0;
  g->state = s;
  return 1;
}

int afb_grammar_accept(void* h, int token) {
  Grammar* g = static_cast<Grammar*>(h);
  const int n = static_cast<int>(g->offsets.size()) - 1;
  if (token < 0 || token >= n) return 0;
  const int64_t b = g->offsets[token], e = g->offsets[token + 1];
  if (e <= b) return 0;
  return afb_grammar_accept_bytes(h, g->bytes.data() + b, static_cast<int>(e - b));
}

// 1 when the bytes accepted so far form a complete JSON document (the end-of-sequence token may be sampled).
int afb_grammar_complete(void* h) { return complete(static_cast<Grammar*>(h)->state) ? 1 : 0; }

int afb_grammar_depth(void* h) { return static_cast<Grammar*>(h)->state.depth; }

}  // extern "C"
