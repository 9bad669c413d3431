// Expression front end: the whitespace-sensitive one-line contraction grammar.
//
// Behaviour follows the reference parser, cogent/src/algs/bases/tc_gen_inputs.py:
//   * '[', ']' and ';' are deleted anywhere in the line (:31-33);
//   * the rest is split on blanks and tokens 0,1,2,3,5,6,8,9 are
//     out-name, "idx,ext,..." list, operator, "sum(idx,ext,..)", left name,
//     left index list, right name, right index list (:48-55);
//   * the output list and the sum list alternate index name and extent (:58-92).
// Lines the reference would crash on (IndexError / ValueError: a name glued to
// its bracket, blanks after commas, no blanks around '*') or accept by accident
// (missing extents) are rejected here with TC_ERR_PARSE instead.
// A line starting with '#' is a comment in the reference's input files
// (cogent/src/generators/tc_gen_etc.py:11) and is not an expression.
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <set>
#include <sstream>

#include "tc_internal.h"

namespace {

std::vector<std::string> split_commas(const std::string& s) {
  std::vector<std::string> out;
  std::string cur;
  for (char c : s) {
    if (c == ',') { out.push_back(cur); cur.clear(); }
    else cur.push_back(c);
  }
  out.push_back(cur);
  return out;
}

bool parse_positive(const std::string& s, int64_t* v) {
  if (s.empty() || s.size() > 18) return false;
  for (char c : s)
    if (!std::isdigit((unsigned char)c)) return false;
  *v = std::strtoll(s.c_str(), nullptr, 10);
  return *v > 0;
}

bool valid_name(const std::string& s) {
  if (s.empty()) return false;
  for (char c : s)
    if (!(std::isalnum((unsigned char)c) || c == '_')) return false;
  return true;
}

bool parse_pairs(const std::string& list, std::vector<std::string>* idx, std::vector<int64_t>* ext,
                 std::string* why, const char* what) {
  std::vector<std::string> parts = split_commas(list);
  if (parts.size() % 2 != 0) {
    *why = std::string(what) + " must alternate index names and extents";
    return false;
  }
  for (size_t i = 0; i < parts.size(); i += 2) {
    int64_t v = 0;
    if (!valid_name(parts[i])) { *why = std::string("bad index name in ") + what; return false; }
    if (!parse_positive(parts[i + 1], &v)) {
      *why = std::string("bad extent '") + parts[i + 1] + "' in " + what;
      return false;
    }
    idx->push_back(parts[i]);
    ext->push_back(v);
  }
  return true;
}

bool parse_names(const std::string& list, std::vector<std::string>* idx, std::string* why, const char* what) {
  std::vector<std::string> parts = split_commas(list);
  for (const std::string& s : parts) {
    if (!valid_name(s)) { *why = std::string("bad index name in ") + what; return false; }
    idx->push_back(s);
  }
  return true;
}

bool contains(const std::vector<std::string>& v, const std::string& s) {
  return std::find(v.begin(), v.end(), s) != v.end();
}

bool has_duplicates(const std::vector<std::string>& v) {
  std::set<std::string> seen(v.begin(), v.end());
  return seen.size() != v.size();
}

void json_list(std::ostringstream& o, const std::vector<std::string>& v) {
  o << "[";
  for (size_t i = 0; i < v.size(); ++i) o << (i ? "," : "") << "\"" << v[i] << "\"";
  o << "]";
}
void json_list(std::ostringstream& o, const std::vector<int64_t>& v) {
  o << "[";
  for (size_t i = 0; i < v.size(); ++i) o << (i ? "," : "") << v[i];
  o << "]";
}

}  // namespace

int tc_parse_expr(const char* line, TcExpr* out, std::string* why) {
  std::string dummy;
  if (!why) why = &dummy;
  if (!line || !out) { *why = "null argument"; return TC_ERR_INVALID_ARG; }
  if (line[0] == '#') { *why = "comment line"; return TC_ERR_PARSE; }

  std::string stripped;
  for (const char* p = line; *p; ++p)
    if (*p != '[' && *p != ']' && *p != ';') stripped.push_back(*p);
  std::vector<std::string> tok;
  {
    std::istringstream in(stripped);
    std::string t;
    while (in >> t) tok.push_back(t);
  }
  if (tok.size() != 10) {
    *why = "expected 10 blank-separated tokens: name [idx,ext,..] op sum(idx,ext,..) * name [idx,..] * name [idx,..]";
    return TC_ERR_PARSE;
  }
  TcExpr e;
  e.out_name = tok[0];
  e.left_name = tok[5];
  e.right_name = tok[8];
  if (!valid_name(e.out_name) || !valid_name(e.left_name) || !valid_name(e.right_name)) {
    *why = "bad tensor name";
    return TC_ERR_PARSE;
  }
  if (tok[2] == "+=") e.op = +1;
  else if (tok[2] == "-=") e.op = -1;
  else if (tok[2] == "=") e.op = 0;
  else { *why = "operator must be +=, -= or ="; return TC_ERR_PARSE; }
  if (tok[4] != "*" || tok[7] != "*") { *why = "operands must be joined by ' * '"; return TC_ERR_PARSE; }
  const std::string& s = tok[3];
  if (s.size() < 6 || s.compare(0, 4, "sum(") != 0 || s.back() != ')') {
    *why = "fourth token must be sum(idx,ext,...)";
    return TC_ERR_PARSE;
  }
  if (!parse_pairs(tok[1], &e.out_idx, &e.out_ext, why, "the output index list")) return TC_ERR_PARSE;
  if (!parse_pairs(s.substr(4, s.size() - 5), &e.sum_idx, &e.sum_ext, why, "sum(...)")) return TC_ERR_PARSE;
  if (!parse_names(tok[6], &e.left_idx, why, "the left operand")) return TC_ERR_PARSE;
  if (!parse_names(tok[9], &e.right_idx, why, "the right operand")) return TC_ERR_PARSE;

  // Structure of a binary contraction.
  if (has_duplicates(e.out_idx) || has_duplicates(e.sum_idx) || has_duplicates(e.left_idx) ||
      has_duplicates(e.right_idx)) {
    *why = "an index appears twice in one tensor";
    return TC_ERR_PARSE;
  }
  for (const std::string& i : e.sum_idx)
    if (contains(e.out_idx, i)) { *why = "index '" + i + "' is both an output and a contraction index"; return TC_ERR_PARSE; }
  for (const std::string& i : e.left_idx)
    if (!contains(e.out_idx, i) && !contains(e.sum_idx, i)) { *why = "left operand uses unknown index '" + i + "'"; return TC_ERR_PARSE; }
  for (const std::string& i : e.right_idx)
    if (!contains(e.out_idx, i) && !contains(e.sum_idx, i)) { *why = "right operand uses unknown index '" + i + "'"; return TC_ERR_PARSE; }
  for (const std::string& i : e.sum_idx)
    if (!contains(e.left_idx, i) || !contains(e.right_idx, i)) {
      *why = "contraction index '" + i + "' must appear in both operands";
      return TC_ERR_PARSE;
    }
  for (const std::string& i : e.out_idx) {
    const bool l = contains(e.left_idx, i), r = contains(e.right_idx, i);
    if (!l && !r) { *why = "output index '" + i + "' appears in no operand"; return TC_ERR_PARSE; }
    if (l && r) { *why = "output index '" + i + "' appears in both operands (batched index)"; return TC_ERR_UNSUPPORTED; }
  }
  *out = e;
  return TC_OK;
}

std::string tc_expr_to_json(const TcExpr& e) {
  std::ostringstream o;
  o << "{\"out\":\"" << e.out_name << "\",\"left\":\"" << e.left_name << "\",\"right\":\"" << e.right_name
    << "\",\"op\":\"" << (e.op > 0 ? "+=" : e.op < 0 ? "-=" : "=") << "\",\"out_idx\":";
  json_list(o, e.out_idx);
  o << ",\"out_ext\":";
  json_list(o, e.out_ext);
  o << ",\"sum_idx\":";
  json_list(o, e.sum_idx);
  o << ",\"sum_ext\":";
  json_list(o, e.sum_ext);
  o << ",\"left_idx\":";
  json_list(o, e.left_idx);
  o << ",\"right_idx\":";
  json_list(o, e.right_idx);
  o << "}";
  return o.str();
}
