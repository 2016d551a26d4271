// Grammar-constrained decoding on the host: a byte-level JSON recogniser and a GBNF (context-free grammar) matcher,
// both driven token by token, and the token mask they induce over a vocabulary.  For every step the sampler asks
// which tokens keep the output a prefix of a sentence of the grammar; the engine masks the others to -inf before
// arg-max / sampling, then feeds the chosen token back.
//
// Counterpart of the reference's JSON grammar mode (zig/pkg/inference/src/pipelines/grammar.zig: a token byte table
// plus a state machine stepped per candidate token).  The recogniser is a deterministic pushdown automaton:
// a stack of open containers (object / array, depth-limited) and a mode that says what may come next.  It is
// strict RFC 8259 JSON (no trailing commas, no leading zeros, escapes checked, control bytes rejected inside
// strings); bytes >= 0x80 inside strings are accepted as UTF-8 payload without validating the sequence.
#include <stdint.h>
#include <string.h>

#include <string>
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

// ---------------------------------------------------------------------------------------------------------
// GBNF: a context-free grammar in the notation llama.cpp popularised (and the reference accepts alongside its JSON
// mode): rules `name ::= alternatives`, literals "...", character classes [a-z0-9_] / [^...], `.`, grouping with
// ( ), and the postfix operators * + ? {m} {m,} {m,n}.  Matching is byte-wise: classes list bytes below 0x80
// (escapes \n \t \r \\ \" \] \xHH); a byte >= 0x80 (UTF-8 payload) matches `.` and negated classes only.
// The matcher is the usual set-of-stacks pushdown simulation: every stack holds the positions still to be
// matched, its top always a terminal; a byte advances the stacks whose top accepts it.
// ---------------------------------------------------------------------------------------------------------
enum ElemType : uint8_t { kEnd, kAlt, kRuleRef, kChar, kCharNot, kCharRngUpper, kCharAlt, kCharAny };
struct Elem { uint8_t type; uint32_t value; };
typedef std::vector<Elem> Rule;  // alternatives separated by kAlt, terminated by kEnd
struct Pos { uint32_t rule, idx; };
typedef std::vector<Pos> Stack;

struct Gbnf {
  std::vector<Rule> rules;
  std::vector<std::string> names;
  uint32_t root = 0;
  std::vector<Stack> stacks;
  std::string error;

  uint32_t rule_id(const std::string& n) {
    for (uint32_t i = 0; i < names.size(); ++i) if (names[i] == n) return i;
    names.push_back(n); rules.emplace_back(); return static_cast<uint32_t>(names.size() - 1);
  }
};

struct GbnfParser {
  Gbnf& g; const char* p; int synth = 0;
  explicit GbnfParser(Gbnf& gg, const char* text) : g(gg), p(text) {}
  bool fail(const std::string& m) { if (g.error.empty()) g.error = m; return false; }
  void ws(bool newlines) {
    for (;;) {
      while (*p == ' ' || *p == '\t' || (newlines && (*p == '\n' || *p == '\r'))) ++p;
      if (*p == '#') { while (*p && *p != '\n') ++p; continue; }
      break;
    }
  }
  static bool name_char(char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '-' || c == '_'; }
  bool parse_name(std::string* out) {
    const char* b = p;
    while (name_char(*p)) ++p;
    if (p == b) return fail("expected a rule name");
    out->assign(b, p);
    return true;
  }
  bool parse_char(uint32_t* out) {
    if (*p == '\\') {
      ++p;
      switch (*p) {
        case 'n': *out = '\n'; ++p; return true;
        case 't': *out = '\t'; ++p; return true;
        case 'r': *out = '\r'; ++p; return true;
        case 'x': {
          uint32_t v = 0;
          for (int i = 0; i < 2; ++i) {
            ++p;
            const char c = *p;
            if (c >= '0' && c <= '9') v = v * 16 + (c - '0');
            else if (c >= 'a' && c <= 'f') v = v * 16 + (c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v = v * 16 + (c - 'A' + 10);
            else return fail("bad \\x escape");
          }
          ++p; *out = v; return true;
        }
        case 0: return fail("dangling backslash");
        default: *out = static_cast<uint8_t>(*p); ++p; return true;  // \\ \" \] \[ \- ...
      }
    }
    if (!*p) return fail("unexpected end of grammar");
    *out = static_cast<uint8_t>(*p); ++p; return true;
  }
  // Wraps the items [from, out.size()) of `out` according to a postfix operator, using synthetic rules.
  bool apply_repeat(Rule& out, size_t from, int lo, int hi /* -1 = unbounded */) {
    Rule item(out.begin() + from, out.end());
    out.resize(from);
    auto new_rule = [&]() { return g.rule_id("_r" + std::to_string(synth++)); };
    for (int i = 0; i < lo; ++i) out.insert(out.end(), item.begin(), item.end());
    if (hi < 0) {  // item*  ==  S ::= item S |
      const uint32_t s = new_rule();
      Rule r(item); r.push_back({kRuleRef, s}); r.push_back({kAlt, 0}); r.push_back({kEnd, 0});
      g.rules[s] = r;
      out.push_back({kRuleRef, s});
    } else {      // up to (hi - lo) optional copies, nested:  O_k ::= item O_{k-1} |
      uint32_t inner = 0; bool have = false;
      for (int i = 0; i < hi - lo; ++i) {
        const uint32_t s = new_rule();
        Rule r(item); if (have) r.push_back({kRuleRef, inner});
        r.push_back({kAlt, 0}); r.push_back({kEnd, 0});
        g.rules[s] = r; inner = s; have = true;
      }
      if (have) out.push_back({kRuleRef, inner});
    }
    return true;
  }
  bool parse_sequence(Rule& out, bool nested) {
    for (;;) {
      ws(nested);
      const size_t from = out.size();
      if (*p == '"') {
        ++p;
        while (*p != '"') {
          uint32_t c;
          if (!parse_char(&c)) return false;
          out.push_back({kChar, c});
        }
        ++p;
        // a multi-byte literal is several items; a postfix operator applies to the whole literal
      } else if (*p == '[') {
        ++p;
        uint8_t t = kChar;
        if (*p == '^') { t = kCharNot; ++p; }
        bool first = true;
        while (*p != ']') {
          uint32_t c;
          if (!parse_char(&c)) return false;
          out.push_back({first ? t : static_cast<uint8_t>(kCharAlt), c});
          first = false;
          if (*p == '-' && p[1] != ']') {
            ++p;
            uint32_t hi;
            if (!parse_char(&hi)) return false;
            out.push_back({kCharRngUpper, hi});
          }
        }
        if (first) return fail("empty character class");
        ++p;
      } else if (*p == '.') {
        ++p; out.push_back({kCharAny, 0});
      } else if (*p == '(') {
        ++p;
        const uint32_t s = g.rule_id("_g" + std::to_string(synth++));
        Rule sub;
        if (!parse_alternates(sub, true)) return false;
        g.rules[s] = sub;
        ws(true);
        if (*p != ')') return fail("expected ')'");
        ++p;
        out.push_back({kRuleRef, s});
      } else if (name_char(*p)) {
        // a name followed by ::= starts the next rule: leave it for the caller
        const char* save = p;
        std::string n;
        if (!parse_name(&n)) return false;
        const char* after = p;
        ws(false);
        if (p[0] == ':' && p[1] == ':' && p[2] == '=') { p = save; return true; }
        p = after;
        out.push_back({kRuleRef, g.rule_id(n)});
      } else {
        return true;  // end of this sequence: '|', ')', newline or end of text
      }
      ws(nested);
      if (*p == '*') { ++p; if (!apply_repeat(out, from, 0, -1)) return false; }
      else if (*p == '+') { ++p; if (!apply_repeat(out, from, 1, -1)) return false; }
      else if (*p == '?') { ++p; if (!apply_repeat(out, from, 0, 1)) return false; }
      else if (*p == '{') {
        ++p;
        int lo = 0, hi = -1; bool any = false;
        while (*p >= '0' && *p <= '9') { lo = lo * 10 + (*p - '0'); ++p; any = true; }
        if (!any) return fail("expected a count in {}");
        if (*p == '}') hi = lo;
        else if (*p == ',') {
          ++p;
          if (*p != '}') { hi = 0; while (*p >= '0' && *p <= '9') { hi = hi * 10 + (*p - '0'); ++p; } }
        } else return fail("bad {} repetition");
        if (*p != '}') return fail("expected '}'");
        ++p;
        if (hi >= 0 && hi < lo) return fail("bad {} bounds");
        if (lo > 256 || hi > 256) return fail("{} repetition too large");
        if (!apply_repeat(out, from, lo, hi)) return false;
      }
    }
  }
  bool parse_alternates(Rule& out, bool nested) {
    if (!parse_sequence(out, nested)) return false;
    ws(nested);
    while (*p == '|') {
      ++p;
      out.push_back({kAlt, 0});
      if (!parse_sequence(out, nested)) return false;
      ws(nested);
    }
    out.push_back({kEnd, 0});
    return true;
  }
  bool parse_all() {
    ws(true);
    while (*p) {
      std::string n;
      if (!parse_name(&n)) return false;
      ws(false);
      if (!(p[0] == ':' && p[1] == ':' && p[2] == '=')) return fail("expected ::= after " + n);
      p += 3;
      Rule r;
      if (!parse_alternates(r, false)) return false;
      const uint32_t id = g.rule_id(n);
      g.rules[id] = r;
      ws(true);
    }
    for (uint32_t i = 0; i < g.rules.size(); ++i)
      if (g.rules[i].empty()) return fail("rule '" + g.names[i] + "' is referenced but never defined");
    return true;
  }
};

inline bool is_char_elem(uint8_t t) { return t == kChar || t == kCharNot || t == kCharAny; }

// Does the terminal at `pos` accept byte c?  Returns the index just past the terminal's elements via *next.
bool match_terminal(const Rule& r, uint32_t idx, uint8_t c, uint32_t* next) {
  const uint8_t t = r[idx].type;
  if (t == kCharAny) { *next = idx + 1; return true; }
  bool found = false;
  uint32_t i = idx;
  do {
    if (i + 1 < r.size() && r[i + 1].type == kCharRngUpper) {
      found = found || (r[i].value <= c && c <= r[i + 1].value);
      i += 2;
    } else {
      found = found || r[i].value == c;
      i += 1;
    }
  } while (i < r.size() && r[i].type == kCharAlt);
  *next = i;
  // positive classes list single bytes, so a UTF-8 payload byte (>= 0x80) only matches one whose range covers it
  return t == kCharNot ? !found : found;
}

// Expands rule references at the top of `stack` until every resulting stack is empty or topped by a terminal.
bool advance_stack(const Gbnf& g, const Stack& stack, std::vector<Stack>& out, int* budget, int depth = 0) {
  // total expansions and nesting are both capped: a left-recursive rule would otherwise expand forever
  if (--*budget < 0 || depth > 512 || stack.size() > 4096) return false;
  if (stack.empty()) { out.push_back(stack); return true; }
  const Pos top = stack.back();
  const Rule& r = g.rules[top.rule];
  const Elem& e = r[top.idx];
  if (e.type == kRuleRef) {
    const Rule& sub = g.rules[e.value];
    uint32_t alt = 0;
    for (;;) {
      Stack ns(stack.begin(), stack.end() - 1);
      // what follows the reference in the current rule
      const uint32_t after = top.idx + 1;
      if (r[after].type != kAlt && r[after].type != kEnd) ns.push_back({top.rule, after});
      if (sub[alt].type != kAlt && sub[alt].type != kEnd) ns.push_back({e.value, alt});
      if (!advance_stack(g, ns, out, budget, depth + 1)) return false;
      while (sub[alt].type != kAlt && sub[alt].type != kEnd) ++alt;
      if (sub[alt].type == kEnd) break;
      ++alt;
    }
    return true;
  }
  if (is_char_elem(e.type)) { out.push_back(stack); return true; }
  return true;  // kAlt / kEnd cannot be on a stack
}

bool gbnf_reset(Gbnf& g) {
  g.stacks.clear();
  const Rule& r = g.rules[g.root];
  int budget = 100000;
  uint32_t alt = 0;
  for (;;) {
    Stack s;
    if (r[alt].type != kAlt && r[alt].type != kEnd) s.push_back({g.root, alt});
    if (!advance_stack(g, s, g.stacks, &budget)) { g.error = "grammar expansion did not terminate (left recursion?)"; return false; }
    while (r[alt].type != kAlt && r[alt].type != kEnd) ++alt;
    if (r[alt].type == kEnd) break;
    ++alt;
  }
  return true;
}

// One byte: the new stack set (empty = rejected).
bool gbnf_step(const Gbnf& g, const std::vector<Stack>& in, uint8_t c, std::vector<Stack>& out) {
  out.clear();
  int budget = 100000;
  for (const Stack& st : in) {
    if (st.empty()) continue;
    const Pos top = st.back();
    const Rule& r = g.rules[top.rule];
    uint32_t next;
    if (!match_terminal(r, top.idx, c, &next)) continue;
    Stack ns(st.begin(), st.end() - 1);
    if (r[next].type != kAlt && r[next].type != kEnd) ns.push_back({top.rule, next});
    if (!advance_stack(g, ns, out, &budget)) return false;
  }
  // identical stacks behave identically: drop duplicates (keeps ambiguous grammars from blowing up)
  for (size_t i = 0; i < out.size(); ++i)
    for (size_t j = i + 1; j < out.size();) {
      bool same = out[i].size() == out[j].size();
      for (size_t k = 0; same && k < out[i].size(); ++k)
        same = out[i][k].rule == out[j][k].rule && out[i][k].idx == out[j][k].idx;
      if (same) out.erase(out.begin() + j); else ++j;
    }
  return !out.empty();
}

struct Grammar {
  int kind = 0;                    // 0 JSON recogniser, 1 GBNF
  JsonState state;
  Gbnf gbnf;
  std::vector<uint8_t> bytes;      // concatenated token byte strings
  std::vector<int64_t> offsets;    // n_tokens + 1
};

thread_local std::string g_grammar_error;

}  // namespace

extern "C" {

void* afb_grammar_json_new(int root_object_only) {
  Grammar* g = new Grammar();
  g->state.root_object_only = root_object_only ? 1 : 0;
  return g;
}

void afb_grammar_free(void* h) { delete static_cast<Grammar*>(h); }

// Compiles a GBNF grammar; `root` names the start rule ("root" when null).  Returns null on a syntax error, an
// undefined rule or a left-recursive grammar; afb_grammar_last_error() then says why.
void* afb_grammar_gbnf_new(const char* text, const char* root) {
  Grammar* g = new Grammar();
  g->kind = 1;
  GbnfParser parser(g->gbnf, text);
  bool ok = parser.parse_all();
  if (ok) {
    const std::string rn = root ? root : "root";
    bool found = false;
    for (uint32_t i = 0; i < g->gbnf.names.size(); ++i)
      if (g->gbnf.names[i] == rn) { g->gbnf.root = i; found = true; }
    if (!found) { g->gbnf.error = "no rule named '" + rn + "'"; ok = false; }
  }
  if (ok) ok = gbnf_reset(g->gbnf);
  if (!ok) {
    g_grammar_error = g->gbnf.error;
    delete g;
    return nullptr;
  }
  return g;
}

const char* afb_grammar_last_error() { return g_grammar_error.c_str(); }

void afb_grammar_reset(void* h) {
  Grammar* g = static_cast<Grammar*>(h);
  if (g->kind == 1) { gbnf_reset(g->gbnf); return; }
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
  if (g->kind == 1) {
    // Most tokens die on their first byte: try each of the 256 first bytes once, then only walk the survivors.
    std::vector<Stack> first[256];
    bool first_ok[256];
    for (int c = 0; c < 256; ++c) first_ok[c] = gbnf_step(g->gbnf, g->gbnf.stacks, static_cast<uint8_t>(c), first[c]);
    std::vector<Stack> cur, nxt;
    for (int t = 0; t < n; ++t) {
      const int64_t b = g->offsets[t], e = g->offsets[t + 1];
      bool ok = e > b && first_ok[g->bytes[b]];
      if (ok && e - b > 1) {
        cur = first[g->bytes[b]];
        for (int64_t i = b + 1; i < e; ++i) {
          if (!gbnf_step(g->gbnf, cur, g->bytes[i], nxt)) { ok = false; break; }
          cur.swap(nxt);
        }
      }
      allowed[t] = ok ? 1 : 0;
      count += ok ? 1 : 0;
    }
    return count;
  }
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
  if (g->kind == 1) {
    std::vector<Stack> cur = g->gbnf.stacks, nxt;
    for (int i = 0; i < n; ++i) {
      if (!gbnf_step(g->gbnf, cur, bytes[i], nxt)) return 0;
      cur.swap(nxt);
    }
    g->gbnf.stacks.swap(cur);
    return 1;
  }
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
int afb_grammar_complete(void* h) {
  Grammar* g = static_cast<Grammar*>(h);
  if (g->kind == 1) {
    for (const Stack& s : g->gbnf.stacks) if (s.empty()) return 1;
    return 0;
  }
  return complete(g->state) ? 1 : 0;
}

int afb_grammar_depth(void* h) { return static_cast<Grammar*>(h)->state.depth; }

}  // extern "C"
