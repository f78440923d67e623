// Grammar-constrained decoding on the host: an EBNF grammar is compiled to a pushdown matcher over Unicode code
// points, the tokenizer's vocabulary to a byte trie, and each decode step asks for the bitmask of tokens that keep the
// output a prefix of a sentence of the grammar.
//
// Grammar text (one rule per `name ::= ...`, `root` is the start rule unless another name is given):
//   "literal" with \n \t \r \\ \" \xHH \uHHHH escapes, [a-z0-9_] and [^...] character classes, . (any character),
//   rule names, ( ... ) groups, | alternatives, postfix * + ? and {m}, {m,}, {m,n} repetition, # comments.
// Repetitions and groups are rewritten into helper rules, so the matcher only sees rules whose alternatives are
// sequences of {character class, rule reference}.
//
// Matching state = a set of stacks of pending grammar positions whose top is a character class (the expansion of
// rule references is done eagerly, with a depth bound that rejects left recursion instead of looping).  A token is
// allowed when its bytes, decoded as UTF-8 after the bytes still pending from earlier tokens, can be consumed from
// some stack; an incomplete trailing sequence is allowed when some class on top can still match a code point with
// that prefix.  The mask is computed by one depth-first walk of the vocabulary trie that carries the stack set, so
// a rejected byte prunes every token below it; masks are cached by a hash of the stack set.
//
// Replaces what the reference links from its xgrammar crate: grammar compilation, the token-mask computation with its
// mask cache, and the per-request matcher (crates/xgrammar, crates/spark-server/src/grammar/{engine,mask_cache}.rs).
#include <algorithm>
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "runtime_api.h"

namespace {

struct Range { uint32_t lo, hi; };

struct CharClass {
  std::vector<Range> ranges;     // sorted, disjoint
  bool negated = false;
  bool matches(uint32_t c) const {
    bool in = false;
    for (const Range& r : ranges)
      if (c >= r.lo && c <= r.hi) { in = true; break; }
    return in != negated;
  }
  // can some code point in [lo, hi] match?
  bool matches_any(uint32_t lo, uint32_t hi) const {
    if (!negated) {
      for (const Range& r : ranges)
        if (r.lo <= hi && r.hi >= lo) return true;
      return false;
    }
    uint32_t cur = lo;                                   // negated: is [lo, hi] fully covered by the ranges?
    for (const Range& r : ranges) {
      if (r.hi < cur) continue;
      if (r.lo > cur) return true;
      cur = r.hi + 1;
      if (cur > hi) return false;
    }
    return cur <= hi;
  }
};

struct Elem { int kind; int id; };                       // kind 0: character class id, kind 1: rule id
using Alt = std::vector<Elem>;
struct Rule { std::string name; std::vector<Alt> alts; };

struct Pos { int rule, alt, idx; };                      // the element alts[alt][idx] of rule
inline bool operator==(const Pos& a, const Pos& b) { return a.rule == b.rule && a.alt == b.alt && a.idx == b.idx; }
using Stack = std::vector<Pos>;

}  // namespace

struct atlas_grammar {
  std::vector<Rule> rules;
  std::vector<CharClass> classes;
  int root = 0;
};

namespace {

// ----------------------------------------------------------------------------- parser
struct Parser {
  const char* p;
  const char* end;
  atlas_grammar* g;
  std::map<std::string, int> ids;
  std::string err;
  int helper = 0;

  explicit Parser(const char* text, atlas_grammar* gr) : p(text), end(text + strlen(text)), g(gr) {}

  int rule_id(const std::string& name) {
    auto it = ids.find(name);
    if (it != ids.end()) return it->second;
    int id = (int)g->rules.size();
    g->rules.push_back(Rule{name, {}});
    ids[name] = id;
    return id;
  }
  int new_helper() { return rule_id("%" + std::to_string(helper++)); }
  int add_class(CharClass c) {
    std::sort(c.ranges.begin(), c.ranges.end(), [](const Range& a, const Range& b) { return a.lo < b.lo; });
    std::vector<Range> merged;
    for (const Range& r : c.ranges) {
      if (!merged.empty() && r.lo <= merged.back().hi + 1) merged.back().hi = std::max(merged.back().hi, r.hi);
      else merged.push_back(r);
    }
    c.ranges = merged;
    g->classes.push_back(c);
    return (int)g->classes.size() - 1;
  }
  void skip_ws(bool newlines) {
    while (p < end) {
      if (*p == '#') { while (p < end && *p != '\n') ++p; }
      else if (*p == ' ' || *p == '\t' || *p == '\r' || (newlines && *p == '\n')) ++p;
      else break;
    }
  }
  static bool name_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '-' || c == '.'; }
  bool fail(const std::string& m) { if (err.empty()) err = m; return false; }

  bool parse_hex(int n, uint32_t* out) {
    uint32_t v = 0;
    for (int i = 0; i < n; ++i) {
      if (p >= end || !isxdigit((unsigned char)*p)) return fail("bad hex escape");
      char c = *p++;
      v = v * 16 + (uint32_t)(isdigit((unsigned char)c) ? c - '0' : (tolower(c) - 'a' + 10));
    }
    *out = v;
    return true;
  }
  // one (possibly escaped, possibly multi-byte) character of a literal or class
  bool parse_char(uint32_t* out) {
    if (p >= end) return fail("unexpected end");
    unsigned char c = (unsigned char)*p;
    if (c == '\\') {
      ++p;
      if (p >= end) return fail("dangling backslash");
      char e = *p++;
      switch (e) {
        case 'n': *out = '\n'; return true;
        case 't': *out = '\t'; return true;
        case 'r': *out = '\r'; return true;
        case 'x': return parse_hex(2, out);
        case 'u': return parse_hex(4, out);
        case 'U': return parse_hex(8, out);
        default: *out = (unsigned char)e; return true;       // \\ \" \] \[ \- \^ ...
      }
    }
    int len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
    if (!len || p + len > end) return fail("bad UTF-8 in grammar");
    uint32_t v = len == 1 ? c : (c & (0xFF >> (len + 1)));
    for (int i = 1; i < len; ++i) v = (v << 6) | ((unsigned char)p[i] & 0x3F);
    p += len;
    *out = v;
    return true;
  }

  // sequence of items up to '|', ')' or end of rule
  bool parse_sequence(Alt* out, bool nested) {
    for (;;) {
      skip_ws(nested);
      if (p >= end || *p == '|' || *p == ')' || (!nested && *p == '\n')) return true;
      Alt item;                                               // the item just parsed (one or more elements)
      if (*p == '"') {
        ++p;
        while (p < end && *p != '"') {
          uint32_t c;
          if (!parse_char(&c)) return false;
          CharClass cc;
          cc.ranges.push_back({c, c});
          item.push_back({0, add_class(cc)});
        }
        if (p >= end) return fail("unterminated string literal");
        ++p;
      } else if (*p == '[') {
        ++p;
        CharClass cc;
        if (p < end && *p == '^') { cc.negated = true; ++p; }
        while (p < end && *p != ']') {
          uint32_t lo, hi;
          if (!parse_char(&lo)) return false;
          hi = lo;
          if (p + 1 < end && *p == '-' && p[1] != ']') {
            ++p;
            if (!parse_char(&hi)) return false;
          }
          if (hi < lo) return fail("reversed range in character class");
          cc.ranges.push_back({lo, hi});
        }
        if (p >= end) return fail("unterminated character class");
        ++p;
        item.push_back({0, add_class(cc)});
      } else if (*p == '.') {
        ++p;
        CharClass cc;
        cc.negated = true;                                    // not in {} = anything
        item.push_back({0, add_class(cc)});
      } else if (*p == '(') {
        ++p;
        int h = new_helper();
        if (!parse_alternatives(h, true)) return false;
        skip_ws(true);
        if (p >= end || *p != ')') return fail("missing )");
        ++p;
        item.push_back({1, h});
      } else if (name_char(*p)) {
        const char* s = p;
        while (p < end && name_char(*p)) ++p;
        std::string name(s, p);
        // a name followed by ::= starts the next rule (only possible at top level after a newline)
        const char* save = p;
        skip_ws(false);
        if (p + 2 < end && p[0] == ':' && p[1] == ':' && p[2] == '=') { p = s; return true; }
        p = save;
        item.push_back({1, rule_id(name)});
      } else {
        return fail(std::string("unexpected character '") + *p + "'");
      }
      // postfix repetition applies to the whole item
      skip_ws(false);
      while (p < end && (*p == '*' || *p == '+' || *p == '?' || *p == '{')) {
        int lo = 0, hi = -1;                                  // hi -1 = unbounded
        if (*p == '*') { ++p; }
        else if (*p == '+') { lo = 1; ++p; }
        else if (*p == '?') { hi = 1; ++p; }
        else {
          ++p;
          lo = 0;
          if (p >= end || !isdigit((unsigned char)*p)) return fail("bad repetition count");
          while (p < end && isdigit((unsigned char)*p)) lo = lo * 10 + (*p++ - '0');
          hi = lo;
          if (p < end && *p == ',') {
            ++p;
            if (p < end && isdigit((unsigned char)*p)) {
              hi = 0;
              while (p < end && isdigit((unsigned char)*p)) hi = hi * 10 + (*p++ - '0');
            } else hi = -1;
          }
          if (p >= end || *p != '}') return fail("missing }");
          ++p;
          if (hi >= 0 && hi < lo) return fail("reversed repetition bounds");
          if (lo > 256 || hi > 256) return fail("repetition bound too large");
        }
        // body rule B ::= item
        int b = new_helper();
        g->rules[b].alts.push_back(item);
        Alt rep;
        for (int i = 0; i < lo; ++i) rep.push_back({1, b});
        if (hi < 0) {                                          // tail T ::= B T | (empty)
          int t = new_helper();
          g->rules[t].alts.push_back(Alt{{1, b}, {1, t}});
          g->rules[t].alts.push_back(Alt{});
          rep.push_back({1, t});
        } else {                                               // nested optionals O_k ::= B O_{k-1} | (empty)
          int prev = -1;
          for (int i = 0; i < hi - lo; ++i) {
            int o = new_helper();
            Alt a{{1, b}};
            if (prev >= 0) a.push_back({1, prev});
            g->rules[o].alts.push_back(a);
            g->rules[o].alts.push_back(Alt{});
            prev = o;
          }
          if (prev >= 0) rep.push_back({1, prev});
        }
        item = rep;
        skip_ws(false);
      }
      out->insert(out->end(), item.begin(), item.end());
    }
  }
  bool parse_alternatives(int rule, bool nested) {
    for (;;) {
      Alt a;
      if (!parse_sequence(&a, nested)) return false;
      g->rules[rule].alts.push_back(a);
      skip_ws(nested);
      if (p < end && *p == '|') { ++p; continue; }
      // a top-level rule may continue on the next line with a leading '|'
      if (!nested) {
        const char* save = p;
        skip_ws(true);
        if (p < end && *p == '|') { ++p; continue; }
        p = save;
      }
      return true;
    }
  }
  bool parse() {
    for (;;) {
      skip_ws(true);
      if (p >= end) break;
      const char* s = p;
      while (p < end && name_char(*p)) ++p;
      if (p == s) return fail("expected a rule name");
      std::string name(s, p);
      skip_ws(false);
      if (p + 2 >= end || p[0] != ':' || p[1] != ':' || p[2] != '=') return fail("expected ::= after '" + name + "'");
      p += 3;
      int id = rule_id(name);
      if (!g->rules[id].alts.empty()) return fail("rule '" + name + "' defined twice");
      if (!parse_alternatives(id, false)) return false;
    }
    for (const Rule& r : g->rules)
      if (r.alts.empty()) return fail("rule '" + r.name + "' is used but never defined");
    return true;
  }
};

// ----------------------------------------------------------------------------- matcher core
constexpr int kMaxDepth = 512;
constexpr size_t kMaxStacks = 4096;

struct StackSet {
  std::vector<Stack> stacks;
  bool overflow = false;
  void add(const Stack& s) {
    for (const Stack& t : stacks)
      if (t == s) return;
    if (stacks.size() >= kMaxStacks) { overflow = true; return; }
    stacks.push_back(s);
  }
};

// expands rule references on top of `s` until the top is a character class (or the stack is empty = sentence complete)
void expand(const atlas_grammar& g, Stack s, StackSet* out, int depth) {
  if (depth > kMaxDepth) { out->overflow = true; return; }
  if (s.empty()) { out->add(s); return; }
  const Pos top = s.back();
  const Elem& e = g.rules[top.rule].alts[top.alt][top.idx];
  if (e.kind == 0) { out->add(s); return; }
  s.pop_back();
  // what follows the reference in its own alternative stays pending below the referenced rule
  if (top.idx + 1 < (int)g.rules[top.rule].alts[top.alt].size()) s.push_back({top.rule, top.alt, top.idx + 1});
  const Rule& r = g.rules[e.id];
  for (int a = 0; a < (int)r.alts.size(); ++a) {
    Stack n = s;
    if (!r.alts[a].empty()) n.push_back({e.id, a, 0});
    expand(g, n, out, depth + 1);
  }
}

// consumes one code point from every stack that can take it
StackSet step(const atlas_grammar& g, const StackSet& in, uint32_t c) {
  StackSet out;
  for (const Stack& s : in.stacks) {
    if (s.empty()) continue;
    const Pos top = s.back();
    const Elem& e = g.rules[top.rule].alts[top.alt][top.idx];
    if (!g.classes[e.id].matches(c)) continue;
    Stack n = s;
    n.pop_back();
    if (top.idx + 1 < (int)g.rules[top.rule].alts[top.alt].size()) n.push_back({top.rule, top.alt, top.idx + 1});
    expand(g, n, &out, 0);
  }
  return out;
}

struct Utf8 {                 // bytes of an incomplete code point
  uint32_t value = 0;
  int remaining = 0;
  int length = 0;             // total bytes of the sequence (bounds the smallest code point it may encode)
};

// Feeds one byte.  Returns -1 on malformed input, 0 when the code point is still incomplete, 1 when *cp is complete.
int feed(Utf8* u, uint8_t b, uint32_t* cp) {
  if (u->remaining == 0) {
    if (b < 0x80) { *cp = b; return 1; }
    if ((b >> 5) == 6) { u->value = b & 0x1F; u->remaining = 1; u->length = 2; return 0; }
    if ((b >> 4) == 14) { u->value = b & 0x0F; u->remaining = 2; u->length = 3; return 0; }
    if ((b >> 3) == 30) { u->value = b & 0x07; u->remaining = 3; u->length = 4; return 0; }
    return -1;
  }
  if ((b >> 6) != 2) return -1;
  u->value = (u->value << 6) | (b & 0x3F);
  if (--u->remaining == 0) {
    static const uint32_t kMin[5] = {0, 0, 0x80, 0x800, 0x10000};
    if (u->value < kMin[u->length] || u->value > 0x10FFFF) return -1;       // overlong or out of range
    *cp = u->value;
    return 1;
  }
  return 0;
}

// can the incomplete sequence still become a code point some stack accepts?
bool partial_ok(const atlas_grammar& g, const StackSet& set, const Utf8& u) {
  if (u.remaining == 0) return true;
  static const uint32_t kMin[5] = {0, 0, 0x80, 0x800, 0x10000};
  uint32_t lo = u.value << (6 * u.remaining);
  const uint32_t hi = std::min(lo | ((1u << (6 * u.remaining)) - 1), 0x10FFFFu);
  lo = std::max(lo, kMin[u.length]);                       // overlong forms are not code points
  if (lo > hi) return false;
  for (const Stack& s : set.stacks) {
    if (s.empty()) continue;
    const Pos top = s.back();
    const Elem& e = g.rules[top.rule].alts[top.alt][top.idx];
    if (g.classes[e.id].matches_any(lo, hi)) return true;
  }
  return false;
}

uint64_t hash_state(const StackSet& set, const Utf8& u) {
  uint64_t h = 1469598103934665603ull ^ ((uint64_t)u.value << 8 | (uint64_t)u.remaining << 4 | (uint64_t)u.length);
  // order independent over stacks, order dependent inside one
  uint64_t acc = 0;
  for (const Stack& s : set.stacks) {
    uint64_t hs = 0x9E3779B97F4A7C15ull;
    for (const Pos& p : s) {
      hs ^= ((uint64_t)p.rule << 40) ^ ((uint64_t)p.alt << 20) ^ (uint64_t)p.idx;
      hs *= 1099511628211ull;
    }
    acc += hs * 0xC2B2AE3D27D4EB4Full;
  }
  return h ^ acc;
}

}  // namespace

// ----------------------------------------------------------------------------- vocabulary trie
struct atlas_vocab {
  struct Node {
    int child[256];
    std::vector<int> tokens;
    Node() { std::fill(child, child + 256, -1); }
  };
  std::vector<Node> nodes;
  std::vector<int> empty_tokens;                       // tokens with no bytes (specials): never allowed by a grammar
  int n_tokens = 0;
};

struct atlas_matcher {
  const atlas_grammar* g;
  const atlas_vocab* v;
  StackSet state;
  Utf8 partial;
  std::vector<std::pair<StackSet, Utf8>> history;      // for rollback
  std::unordered_map<uint64_t, std::vector<uint32_t>> cache;
  bool failed = false;
};

namespace {

void walk(const atlas_matcher* m, int node, const StackSet& set, const Utf8& u, std::vector<uint32_t>* bits) {
  const atlas_vocab::Node& n = m->v->nodes[node];
  if (node != 0 && !n.tokens.empty() && partial_ok(*m->g, set, u))
    for (int t : n.tokens) (*bits)[t >> 5] |= 1u << (t & 31);
  for (int b = 0; b < 256; ++b) {
    const int c = n.child[b];
    if (c < 0) continue;
    Utf8 nu = u;
    uint32_t cp = 0;
    const int r = feed(&nu, (uint8_t)b, &cp);
    if (r < 0) continue;
    if (r == 0) {
      if (!partial_ok(*m->g, set, nu)) continue;
      walk(m, c, set, nu, bits);
    } else {
      StackSet next = step(*m->g, set, cp);
      if (next.stacks.empty()) continue;
      walk(m, c, next, Utf8{}, bits);
    }
  }
}

}  // namespace

extern "C" {

atlas_grammar* atlas_grammar_compile(const char* text, const char* root, char* err, int errcap) {
  std::unique_ptr<atlas_grammar> g(new atlas_grammar());
  Parser ps(text, g.get());
  bool ok = ps.parse();
  if (ok) {
    auto it = ps.ids.find(root && *root ? root : "root");
    if (it == ps.ids.end()) ok = ps.fail(std::string("no rule named '") + (root && *root ? root : "root") + "'");
    else g->root = it->second;
  }
  if (!ok) {
    if (err && errcap > 0) snprintf(err, (size_t)errcap, "%s", ps.err.c_str());
    return nullptr;
  }
  return g.release();
}
void atlas_grammar_destroy(atlas_grammar* g) { delete g; }
int atlas_grammar_num_rules(const atlas_grammar* g) { return (int)g->rules.size(); }

atlas_vocab* atlas_vocab_create(const uint8_t* bytes, const int64_t* offsets, int n_tokens) {
  atlas_vocab* v = new atlas_vocab();
  v->n_tokens = n_tokens;
  v->nodes.emplace_back();
  for (int t = 0; t < n_tokens; ++t) {
    const int64_t lo = offsets[t], hi = offsets[t + 1];
    if (hi <= lo) { v->empty_tokens.push_back(t); continue; }
    int cur = 0;
    for (int64_t i = lo; i < hi; ++i) {
      int nxt = v->nodes[cur].child[bytes[i]];
      if (nxt < 0) {
        nxt = (int)v->nodes.size();
        v->nodes[cur].child[bytes[i]] = nxt;
        v->nodes.emplace_back();
      }
      cur = nxt;
    }
    v->nodes[cur].tokens.push_back(t);
  }
  return v;
}
void atlas_vocab_destroy(atlas_vocab* v) { delete v; }
int atlas_vocab_num_nodes(const atlas_vocab* v) { return (int)v->nodes.size(); }

atlas_matcher* atlas_matcher_create(const atlas_grammar* g, const atlas_vocab* v) {
  atlas_matcher* m = new atlas_matcher();
  m->g = g;
  m->v = v;
  const Rule& r = g->rules[g->root];
  for (int a = 0; a < (int)r.alts.size(); ++a) {
    Stack s;
    if (!r.alts[a].empty()) s.push_back({g->root, a, 0});
    expand(*g, s, &m->state, 0);
  }
  m->failed = m->state.overflow;
  return m;
}
void atlas_matcher_destroy(atlas_matcher* m) { delete m; }

// 1 when the text so far is a complete sentence (no pending bytes and some stack is empty)
int atlas_matcher_can_end(const atlas_matcher* m) {
  if (m->partial.remaining) return 0;
  for (const Stack& s : m->state.stacks)
    if (s.empty()) return 1;
  return 0;
}
// 1 when nothing but the end of the text can follow
int atlas_matcher_exhausted(const atlas_matcher* m) {
  for (const Stack& s : m->state.stacks)
    if (!s.empty()) return 0;
  return 1;
}

// Fills `bits` (n_words 32-bit words, bit t = token t allowed).  Returns the number of allowed tokens, -1 when the
// grammar overflowed its bounds (left recursion or too many simultaneous parses).
int atlas_matcher_mask(atlas_matcher* m, uint32_t* bits, int n_words) {
  if (m->failed) return -1;
  const int need = (m->v->n_tokens + 31) / 32;
  if (n_words < need) return -2;
  const uint64_t key = hash_state(m->state, m->partial);
  auto it = m->cache.find(key);
  if (it == m->cache.end()) {
    std::vector<uint32_t> b((size_t)need, 0u);
    walk(m, 0, m->state, m->partial, &b);
    if (m->cache.size() > 512) m->cache.clear();
    it = m->cache.emplace(key, std::move(b)).first;
  }
  memcpy(bits, it->second.data(), (size_t)need * 4);
  memset(bits + need, 0, (size_t)(n_words - need) * 4);
  int count = 0;
  for (int i = 0; i < need; ++i) count += __builtin_popcount(it->second[i]);
  return count;
}

// Consumes the bytes of one token.  Returns 1 and advances, or 0 and leaves the state untouched.
int atlas_matcher_accept_bytes(atlas_matcher* m, const uint8_t* bytes, int n) {
  if (m->failed || n <= 0) return 0;
  StackSet set = m->state;
  Utf8 u = m->partial;
  for (int i = 0; i < n; ++i) {
    uint32_t cp = 0;
    const int r = feed(&u, bytes[i], &cp);
    if (r < 0) return 0;
    if (r == 1) {
      set = step(*m->g, set, cp);
      if (set.overflow) { m->failed = true; return 0; }
      if (set.stacks.empty()) return 0;
      u = Utf8{};
    }
  }
  if (!partial_ok(*m->g, set, u)) return 0;
  m->history.emplace_back(m->state, m->partial);
  if (m->history.size() > 64) m->history.erase(m->history.begin());
  m->state = std::move(set);
  m->partial = u;
  return 1;
}

// Undoes the last `n` accepted tokens (speculative decoding rejects drafts); returns how many were undone.
int atlas_matcher_rollback(atlas_matcher* m, int n) {
  int done = 0;
  while (done < n && !m->history.empty()) {
    m->state = std::move(m->history.back().first);
    m->partial = m->history.back().second;
    m->history.pop_back();
    ++done;
  }
  return done;
}

int atlas_matcher_num_stacks(const atlas_matcher* m) { return (int)m->state.stacks.size(); }

}  // extern "C"
