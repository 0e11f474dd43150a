// Signature scan of Triton IR text.
//
// The reference lowers the whole module to Metal source
// (Sources/TritonMetalCore/MSLEmitter.swift).  This library holds precompiled
// sm_100a kernels instead, so all it needs from the IR is what the launch ABI
// does not carry: the entry name, the argument list (presence and order - real
// Triton drops unit-stride arguments, and the Swift and Python attn_fwd orders
// differ), the element type and the BLOCK shape that gives the launch grid its
// meaning.  This is a scanner over the `tt.func` header and the first `tt.dot`,
// not a parser of the body, and certainly not a compiler.
//
// Error wording follows CoreError.description
// (Sources/TritonMetalCore/IR/TritonIR.swift:383-400).

#include "tm_core.h"

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <sstream>

namespace tmc {

const char* kernel_entry_name(KernelId id) {
  switch (id) {
    case KernelId::Matmul: return "matmul_kernel";
    case KernelId::AttnFwd: return "attn_fwd";
    case KernelId::AttnBwdPreprocess: return "attn_bwd_preprocess";
    case KernelId::AttnBwdDq: return "attn_bwd_dq";
    case KernelId::AttnBwdDkdv: return "attn_bwd_dkdv";
    case KernelId::VecCopy: return "copy_kernel";
    case KernelId::VecAdd: return "add_kernel";
    case KernelId::VecMul: return "mul_kernel";
    case KernelId::ScaleBias: return "scale_bias_kernel";
    case KernelId::Softmax: return "softmax_kernel";
    case KernelId::SaeEncode: return "sae_encode_kernel";
    default: return "?";
  }
}

namespace {

struct Loc { int line = 1, col = 1; };

Loc loc_of(const std::string& s, size_t pos) {
  Loc l;
  for (size_t i = 0; i < pos && i < s.size(); ++i) {
    if (s[i] == '\n') { l.line++; l.col = 1; } else { l.col++; }
  }
  return l;
}

std::string loc_str(Loc l) {
  return "line " + std::to_string(l.line) + ", col " + std::to_string(l.col);
}

bool ident_char(char c) { return std::isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$'; }

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace((unsigned char)s[a])) a++;
  while (b > a && std::isspace((unsigned char)s[b - 1])) b--;
  return s.substr(a, b - a);
}

std::string lower(std::string s) {
  for (auto& c : s) c = (char)std::tolower((unsigned char)c);
  return s;
}

// Ops of the reference's supported IR subset (IR/Parser.swift) that may appear
// in a module handed to this library.  Anything in the tt dialect outside this
// set is reported the way the reference reports it.
const std::set<std::string>& known_tt_ops() {
  static const std::set<std::string> ops = {
      "tt.func", "tt.return", "tt.get_program_id", "tt.get_num_programs", "tt.make_range",
      "tt.splat", "tt.expand_dims", "tt.broadcast", "tt.addptr", "tt.load", "tt.store",
      "tt.dot", "tt.trans", "tt.reduce", "tt.reduce.return", "tt.atomic_rmw", "tt.atomic_cas",
      "tt.exp", "tt.log", "tt.sin", "tt.cos", "tt.sqrt", "tt.ptr", "tt.divisibility",
      "tt.call", "tt.bitcast", "tt.fp_to_fp", "tt.reshape", "tt.precise_sqrt",
      "tt.precise_divf", "tt.mulhiui", "tt.clampf", "tt.int_to_ptr", "tt.ptr_to_int",
      "tt.contiguity", "tt.constancy", "tt.pointer_range", "tt.assert", "tt.print"};
  return ops;
}

Role role_from_name(KernelId id, const std::string& raw) {
  std::string n = lower(raw);
  if (id == KernelId::Matmul) {
    static const std::map<std::string, Role> m = {
        {"a_ptr", Role::A}, {"b_ptr", Role::B}, {"c_ptr", Role::C}, {"a", Role::A}, {"b", Role::B},
        {"c", Role::C}, {"m", Role::M}, {"n", Role::N}, {"k", Role::K},
        {"stride_am", Role::StrideAm}, {"stride_ak", Role::StrideAk}, {"stride_bk", Role::StrideBk},
        {"stride_bn", Role::StrideBn}, {"stride_cm", Role::StrideCm}, {"stride_cn", Role::StrideCn}};
    auto it = m.find(n);
    return it == m.end() ? Role::Unknown : it->second;
  }
  static const std::map<std::string, Role> m = {
      {"q", Role::Q}, {"k", Role::Kt}, {"v", Role::V}, {"o", Role::O}, {"out", Role::O},
      {"do", Role::DO}, {"dq", Role::DQ}, {"dk", Role::DK}, {"dv", Role::DV}, {"l", Role::L},
      {"lse", Role::L}, {"m", Role::L}, {"d", Role::Delta}, {"delta", Role::Delta},
      {"sm_scale", Role::SmScale}, {"stride_head", Role::StrideHead},
      {"stride_seq", Role::StrideSeq}, {"stride_lse", Role::StrideLse}, {"n_ctx", Role::NCtx}};
  auto it = m.find(n);
  return it == m.end() ? Role::Unknown : it->second;
}

// Positional roles when the IR names its arguments %arg0, %arg1, ...
bool assign_positional(KernelDesc& d, std::string& err) {
  auto& a = d.args;
  auto fail = [&](const std::string& why) {
    err = std::string("lowering error at line 0, col 0: ") + kernel_entry_name(d.id) + " " + why;
    return false;
  };
  auto set = [&](std::initializer_list<Role> roles) {
    size_t i = 0;
    for (Role r : roles) a[i++].role = r;
  };
  switch (d.id) {
    case KernelId::Matmul:
      if (a.size() == 12) {
        set({Role::A, Role::B, Role::C, Role::M, Role::N, Role::K, Role::StrideAm, Role::StrideAk,
             Role::StrideBk, Role::StrideBn, Role::StrideCm, Role::StrideCn});
      } else if (a.size() == 9) {
        // Real Triton folds the unit strides away (python/examples/matmul.py passes
        // K,1,N,1,N,1): what remains is the three row strides.
        set({Role::A, Role::B, Role::C, Role::M, Role::N, Role::K, Role::StrideAm, Role::StrideBk,
             Role::StrideCm});
      } else {
        return fail("takes 12 arguments (or 9 with unit strides folded), found " +
                    std::to_string(a.size()));
      }
      return true;
    case KernelId::AttnFwd:
      if (a.size() == 8) {
        set({Role::Q, Role::Kt, Role::V, Role::O, Role::SmScale, Role::StrideHead, Role::StrideSeq,
             Role::NCtx});
      } else if (a.size() == 10 && !a[4].is_pointer) {
        // Sources/TritonMetalBench/AttentionKernel.swift:75-78 with emitStats.
        set({Role::Q, Role::Kt, Role::V, Role::O, Role::SmScale, Role::StrideHead, Role::StrideSeq,
             Role::NCtx, Role::L, Role::StrideLse});
      } else if (a.size() == 10) {
        // python/examples/attention_training.py:38.
        set({Role::Q, Role::Kt, Role::V, Role::O, Role::L, Role::SmScale, Role::StrideHead,
             Role::StrideSeq, Role::StrideLse, Role::NCtx});
      } else {
        return fail("takes 8 or 10 arguments, found " + std::to_string(a.size()));
      }
      return true;
    case KernelId::AttnBwdPreprocess:
      if (a.size() != 7) return fail("takes 7 arguments, found " + std::to_string(a.size()));
      set({Role::O, Role::DO, Role::Delta, Role::StrideHead, Role::StrideSeq, Role::StrideLse,
           Role::NCtx});
      return true;
    case KernelId::AttnBwdDq:
      if (a.size() != 12) return fail("takes 12 arguments, found " + std::to_string(a.size()));
      set({Role::Q, Role::Kt, Role::V, Role::DO, Role::DQ, Role::L, Role::Delta, Role::SmScale,
           Role::StrideHead, Role::StrideSeq, Role::StrideLse, Role::NCtx});
      return true;
    case KernelId::AttnBwdDkdv:
      if (a.size() != 13) return fail("takes 13 arguments, found " + std::to_string(a.size()));
      set({Role::Q, Role::Kt, Role::V, Role::DO, Role::DK, Role::DV, Role::L, Role::Delta,
           Role::SmScale, Role::StrideHead, Role::StrideSeq, Role::StrideLse, Role::NCtx});
      return true;
    // The one-dimensional kernels are matched by position only: pointers first, then scalars.
    case KernelId::VecCopy:
      if (a.size() != 3) return fail("takes 3 arguments (in, out, n), found " + std::to_string(a.size()));
      set({Role::In0, Role::Out, Role::Count});
      return true;
    case KernelId::VecAdd:
    case KernelId::VecMul:
      if (a.size() != 4) return fail("takes 4 arguments (a, b, out, n), found " + std::to_string(a.size()));
      set({Role::In0, Role::In1, Role::Out, Role::Count});
      return true;
    case KernelId::ScaleBias:
      if (a.size() != 5)
        return fail("takes 5 arguments (in, out, scale, bias, n), found " + std::to_string(a.size()));
      set({Role::In0, Role::Out, Role::Scale, Role::Bias, Role::Count});
      return true;
    case KernelId::Softmax:
      if (a.size() != 5)
        return fail("takes 5 arguments (in, out, in_row_stride, out_row_stride, n_cols), found " +
                    std::to_string(a.size()));
      set({Role::In0, Role::Out, Role::StrideIn, Role::StrideOut, Role::NCols});
      return true;
    case KernelId::SaeEncode:
      if (a.size() != 7)
        return fail("takes 7 arguments (x, w, bias, out, M, D, F), found " + std::to_string(a.size()));
      set({Role::A, Role::B, Role::BiasVec, Role::C, Role::M, Role::K, Role::N});
      return true;
    default:
      return fail("is not a known entry");
  }
}

// Required roles, each present once, with the pointer / scalar kind and the statistic and scale
// types the kernels expect.  Shared by the IR scan and by parse_descriptor, so a descriptor that
// did not come from tm_emit_msl (truncated, stale, edited) is refused instead of trusted.
bool check_roles(const KernelDesc& d, std::string& err) {
  // Required roles and their kinds.
  auto has = [&](Role r) {
    for (auto& a : d.args) if (a.role == r) return true;
    return false;
  };
  std::vector<Role> need;
  switch (d.id) {
    case KernelId::Matmul: need = {Role::A, Role::B, Role::C, Role::M, Role::N, Role::K}; break;
    case KernelId::AttnFwd:
      need = {Role::Q, Role::Kt, Role::V, Role::O, Role::SmScale, Role::StrideHead, Role::StrideSeq,
              Role::NCtx};
      break;
    case KernelId::AttnBwdPreprocess:
      need = {Role::O, Role::DO, Role::Delta, Role::StrideHead, Role::StrideSeq, Role::StrideLse,
              Role::NCtx};
      break;
    case KernelId::AttnBwdDq:
      need = {Role::Q, Role::Kt, Role::V, Role::DO, Role::DQ, Role::L, Role::Delta, Role::SmScale,
              Role::StrideHead, Role::StrideSeq, Role::StrideLse, Role::NCtx};
      break;
    case KernelId::AttnBwdDkdv:
      need = {Role::Q, Role::Kt, Role::V, Role::DO, Role::DK, Role::DV, Role::L, Role::Delta,
              Role::SmScale, Role::StrideHead, Role::StrideSeq, Role::StrideLse, Role::NCtx};
      break;
    case KernelId::VecCopy: need = {Role::In0, Role::Out, Role::Count}; break;
    case KernelId::VecAdd: case KernelId::VecMul: need = {Role::In0, Role::In1, Role::Out, Role::Count}; break;
    case KernelId::ScaleBias: need = {Role::In0, Role::Out, Role::Scale, Role::Bias, Role::Count}; break;
    case KernelId::Softmax: need = {Role::In0, Role::Out, Role::StrideIn, Role::StrideOut, Role::NCols}; break;
    case KernelId::SaeEncode:
      need = {Role::A, Role::B, Role::BiasVec, Role::C, Role::M, Role::K, Role::N};
      break;
    default: break;
  }
  {
    std::set<int> once;
    for (auto& a : d.args) {
      if (a.role != Role::Unknown && !once.insert((int)a.role).second) {
        err = std::string("lowering error at line 0, col 0: ") + kernel_entry_name(d.id) +
              " has two arguments with the same role (" + std::to_string((int)a.role) + ")";
        return false;
      }
    }
  }
  for (Role r : need) {
    if (!has(r)) {
      err = std::string("lowering error at line 0, col 0: ") + kernel_entry_name(d.id) +
            " is missing a required argument (role " + std::to_string((int)r) + ")";
      return false;
    }
  }
  for (auto& a : d.args) {
    bool want_ptr = false;
    switch (a.role) {
      case Role::A: case Role::B: case Role::C: case Role::Q: case Role::Kt: case Role::V:
      case Role::O: case Role::DO: case Role::DQ: case Role::DK: case Role::DV: case Role::L:
      case Role::Delta: case Role::In0: case Role::In1: case Role::Out: case Role::BiasVec:
        want_ptr = true; break;
      default: break;
    }
    if (want_ptr != a.is_pointer) {
      err = std::string("lowering error at line 0, col 0: argument ") + std::to_string(a.index) +
            " ('" + a.name + "') of " + kernel_entry_name(d.id) + " should be a " +
            (want_ptr ? "pointer" : "scalar");
      return false;
    }
    if ((a.role == Role::L || a.role == Role::Delta) && a.dtype != "f32") {
      err = "unsupported type '" + a.dtype + "' at line 0, col 0";
      return false;
    }
    if ((a.role == Role::SmScale || a.role == Role::Scale || a.role == Role::Bias) && a.dtype != "f32") {
      err = "unsupported type '" + a.dtype + "' at line 0, col 0";
      return false;
    }
  }
  return true;
}


bool assign_roles(KernelDesc& d, std::string& err) {
  // By name when every argument has a recognisable role name, else by position.
  bool all_named = !d.args.empty() && !is_rowwise(d.id) && d.id != KernelId::SaeEncode;
  std::set<int> seen;
  for (auto& a : d.args) {
    Role r = role_from_name(d.id, a.name);
    if (r == Role::Unknown || seen.count((int)r)) { all_named = false; break; }
    seen.insert((int)r);
  }
  if (all_named) {
    for (auto& a : d.args) a.role = role_from_name(d.id, a.name);
  } else if (!assign_positional(d, err)) {
    return false;
  }
  return check_roles(d, err);
}

// Split "a, b<c, d>, e {x, y}" on the commas at nesting depth 0.
std::vector<std::pair<std::string, size_t>> split_top(const std::string& s, size_t base) {
  std::vector<std::pair<std::string, size_t>> out;
  int depth = 0;
  size_t start = 0;
  for (size_t i = 0; i <= s.size(); ++i) {
    char c = i < s.size() ? s[i] : ',';
    if (c == '<' || c == '(' || c == '{' || c == '[') depth++;
    else if (c == '>' || c == ')' || c == '}' || c == ']') depth--;
    if (c == ',' && depth == 0) {
      std::string piece = trim(s.substr(start, i - start));
      if (!piece.empty()) out.push_back({piece, base + start});
      start = i + 1;
    }
  }
  return out;
}

bool parse_tensor_2d(const std::string& s, size_t from, int& d0, int& d1, std::string& elt,
                     size_t* end_pos) {
  // finds the next "tensor<AxBxT>" with exactly two integer extents at or after `from`
  size_t pos = from;
  while ((pos = s.find("tensor<", pos)) != std::string::npos) {
    size_t p = pos + 7;
    std::vector<int> dims;
    while (p < s.size() && std::isdigit((unsigned char)s[p])) {
      int v = 0;
      while (p < s.size() && std::isdigit((unsigned char)s[p])) v = v * 10 + (s[p++] - '0');
      if (p < s.size() && s[p] == 'x') { dims.push_back(v); p++; } else { dims.clear(); break; }
    }
    size_t q = p;
    while (q < s.size() && ident_char(s[q])) q++;
    std::string e = s.substr(p, q - p);
    if (dims.size() == 2 && q < s.size() && s[q] == '>' && (e == "f32" || e == "f16" || e == "bf16")) {
      d0 = dims[0]; d1 = dims[1]; elt = e;
      if (end_pos) *end_pos = q;
      return true;
    }
    pos = pos + 7;
  }
  return false;
}

}  // namespace

bool scan_module(const std::string& ttir, int num_simdgroups, std::vector<KernelDesc>& out,
                 std::string& error) {
  out.clear();
  // 1. an op of the tt dialect outside the supported subset is refused by name.
  for (size_t pos = 0; (pos = ttir.find("tt.", pos)) != std::string::npos;) {
    bool boundary = pos == 0 || !(ident_char(ttir[pos - 1]) || ttir[pos - 1] == '!' ||
                                  ttir[pos - 1] == '%' || ttir[pos - 1] == '@' || ttir[pos - 1] == '#');
    size_t e = pos;
    while (e < ttir.size() && ident_char(ttir[e])) e++;
    std::string op = ttir.substr(pos, e - pos);
    while (!op.empty() && op.back() == '.') op.pop_back();
    if (boundary && !known_tt_ops().count(op)) {
      error = "unsupported op '" + op + "' at " + loc_str(loc_of(ttir, pos)) +
              ": libtmcuda does not implement this operation (it holds precompiled sm_100a kernels "
              "for matmul_kernel and the attn_* entries, not a Triton IR compiler)";
      return false;
    }
    pos = e > pos ? e : pos + 3;
  }

  // 2. every tt.func header.
  size_t pos = 0;
  while ((pos = ttir.find("tt.func", pos)) != std::string::npos) {
    size_t header = pos;
    pos += 7;
    size_t at = ttir.find('@', pos);
    if (at == std::string::npos) break;
    size_t ne = at + 1;
    while (ne < ttir.size() && ident_char(ttir[ne])) ne++;
    std::string name = ttir.substr(at + 1, ne - at - 1);
    size_t open = ttir.find('(', ne);
    if (open == std::string::npos) {
      error = "parse error at " + loc_str(loc_of(ttir, ne)) + ": expected '(' after the function name";
      return false;
    }
    int depth = 0;
    size_t close = open;
    for (; close < ttir.size(); ++close) {
      if (ttir[close] == '(') depth++;
      else if (ttir[close] == ')' && --depth == 0) break;
    }
    if (close >= ttir.size()) {
      error = "parse error at " + loc_str(loc_of(ttir, open)) + ": unterminated argument list";
      return false;
    }
    KernelDesc d;
    bool known = false;
    for (int i = 0; i < (int)KernelId::Count; ++i) {
      if (name == kernel_entry_name((KernelId)i)) { d.id = (KernelId)i; known = true; }
    }
    if (!known) {
      error = "unimplemented: kernel '" + name + "' at " + loc_str(loc_of(ttir, header)) +
              " has no sm_100a implementation in libtmcuda (available: add_kernel, attn_bwd_dkdv, "
              "attn_bwd_dq, attn_bwd_preprocess, attn_fwd, copy_kernel, matmul_kernel, mul_kernel, "
              "sae_encode_kernel, scale_bias_kernel, softmax_kernel)";
      return false;
    }
    auto pieces = split_top(ttir.substr(open + 1, close - open - 1), open + 1);
    int index = 0;
    for (auto& pr : pieces) {
      const std::string& piece = pr.first;
      ArgInfo a;
      a.index = index++;
      size_t colon = piece.find(':');
      if (piece.empty() || piece[0] != '%' || colon == std::string::npos) {
        error = "parse error at " + loc_str(loc_of(ttir, pr.second)) +
                ": expected '%name: type' in the argument list";
        return false;
      }
      a.name = trim(piece.substr(1, colon - 1));
      std::string ty = trim(piece.substr(colon + 1));
      size_t brace = ty.find('{');
      if (brace != std::string::npos) ty = trim(ty.substr(0, brace));
      if (ty.rfind("!tt.ptr<", 0) == 0) {
        a.is_pointer = true;
        size_t gt = ty.find_first_of(",>", 8);
        a.dtype = trim(ty.substr(8, gt == std::string::npos ? std::string::npos : gt - 8));
      } else {
        a.dtype = ty;
      }
      if (a.dtype == "f64") {
        error = "unsupported type 'f64' at " + loc_str(loc_of(ttir, pr.second)) +
                ": the launch ABI carries 32-bit scalars and i64 only";
        return false;
      }
      d.args.push_back(a);
    }
    if (!assign_roles(d, error)) return false;

    // element type: the pointee of the first operand.
    const std::string& e0 = d.args[0].dtype;
    if (e0 == "f32") d.elt = Elt::F32;
    else if (e0 == "f16") d.elt = Elt::F16;
    else if (e0 == "bf16") d.elt = Elt::BF16;
    else {
      error = "unsupported type '" + e0 + "' at " + loc_str(loc_of(ttir, header));
      return false;
    }
    for (auto& a : d.args) {
      bool data_ptr = a.is_pointer && a.role != Role::L && a.role != Role::Delta;
      if (data_ptr && a.dtype != e0) {
        error = "lowering error at " + loc_str(loc_of(ttir, header)) +
                ": tt.dot operands and result must share one element type, found '" + e0 +
                "' and '" + a.dtype + "'";
        return false;
      }
    }

    // block shape: from the first tt.dot of this function, else the first rank-2 tensor.
    size_t next_func = ttir.find("tt.func", close);
    std::string body = ttir.substr(close, next_func == std::string::npos ? std::string::npos
                                                                         : next_func - close);
    if (is_rowwise(d.id)) {
      // BLOCK is the extent of the first tt.make_range; the body must hold the operations the
      // precompiled kernel of that name performs (a same-named kernel doing something else is
      // refused rather than silently replaced).
      if (d.elt != Elt::F32) {
        error = "unsupported type '" + e0 + "' at " + loc_str(loc_of(ttir, header)) + ": " +
                kernel_entry_name(d.id) + " is precompiled for f32 only";
        return false;
      }
      size_t mr = body.find("tt.make_range");
      size_t endk = mr == std::string::npos ? mr : body.find("end = ", mr);
      int block = endk == std::string::npos ? 0 : std::atoi(body.c_str() + endk + 6);
      if (block <= 0 || block > 65536) {
        error = "lowering error at " + loc_str(loc_of(ttir, header)) + ": " + kernel_entry_name(d.id) +
                " needs a tt.make_range {end = BLOCK} with 0 < BLOCK <= 65536";
        return false;
      }
      auto has_op = [&](const char* op) { return body.find(op) != std::string::npos; };
      bool ok_body = has_op("tt.load") && has_op("tt.store");
      switch (d.id) {
        case KernelId::VecCopy: ok_body = ok_body && !has_op("arith.addf") && !has_op("arith.mulf"); break;
        case KernelId::VecAdd: ok_body = ok_body && has_op("arith.addf") && !has_op("arith.mulf"); break;
        case KernelId::VecMul: ok_body = ok_body && has_op("arith.mulf") && !has_op("arith.addf"); break;
        case KernelId::ScaleBias: ok_body = ok_body && has_op("arith.mulf") && has_op("arith.addf"); break;
        case KernelId::Softmax:
          ok_body = ok_body && has_op("tt.reduce") && has_op("math.exp") && has_op("arith.divf") &&
                    has_op("arith.maxnumf");
          break;
        default: break;
      }
      if (!ok_body) {
        error = "unimplemented: the body of '" + name + "' at " + loc_str(loc_of(ttir, header)) +
                " is not the computation libtmcuda's precompiled " + kernel_entry_name(d.id) + " performs";
        return false;
      }
      d.block_m = block;
      d.threads = std::min(1024, std::max(32, num_simdgroups <= 0 ? 32 : num_simdgroups * 32));
      out.push_back(d);
      pos = close;
      continue;
    }
    if (d.id == KernelId::SaeEncode) {
      auto has_op = [&](const char* op) { return body.find(op) != std::string::npos; };
      if (d.elt != Elt::F32) {
        error = "unsupported type '" + e0 + "' at " + loc_str(loc_of(ttir, header)) +
                ": sae_encode_kernel is precompiled for f32 only";
        return false;
      }
      if (!(has_op("tt.dot") && has_op("arith.addf") && has_op("arith.maximumf") && has_op("tt.store"))) {
        error = "unimplemented: the body of '" + name + "' at " + loc_str(loc_of(ttir, header)) +
                " is not the computation libtmcuda's precompiled sae_encode_kernel performs "
                "(relu(x @ w + bias))";
        return false;
      }
    }
    size_t dot = body.find("tt.dot");
    int r0 = 0, r1 = 0;
    std::string te;
    if (dot != std::string::npos) {
      size_t colon = body.find(" : ", dot);
      size_t p1 = 0, p2 = 0;
      int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
      if (colon != std::string::npos && parse_tensor_2d(body, colon, a0, a1, te, &p1) &&
          parse_tensor_2d(body, p1, b0, b1, te, &p2)) {
        // lhs [a0 x a1] * rhs [b0 x b1]
        if (d.id == KernelId::Matmul || d.id == KernelId::SaeEncode) { d.block_m = a0; d.block_k = a1; d.block_n = b1; }
        else if (d.id == KernelId::AttnBwdDkdv) { d.block_n = a0; d.head_dim = a1; d.block_m = b1; }
        else { d.block_m = a0; d.head_dim = a1; d.block_n = b1; }
      }
    } else if (parse_tensor_2d(body, 0, r0, r1, te, nullptr)) {
      d.block_m = r0; d.head_dim = r1;
    }
    d.threads = std::min(1024, std::max(32, num_simdgroups <= 0 ? 32 : num_simdgroups * 32));
    // an optional attribute on the function selects causal masking
    // (`tt.func @attn_fwd(...) attributes {tm.causal = true} {`): everything between the
    // argument list and the first SSA value of the body is the attribute dictionary.
    size_t first_value = body.find('%');
    if (body.substr(0, first_value).find("tm.causal = true") != std::string::npos) d.causal = 1;
    out.push_back(d);
    pos = close;
  }
  if (out.empty()) {
    error = "parse error at line 1, col 1: module contains no tt.func to lower";
    return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// Descriptor text (what tm_emit_msl returns and tm_compile_msl consumes)
// ---------------------------------------------------------------------------

static const char* kMagic = "// tmcuda kernel descriptor v1";

std::string descriptor_text(const std::vector<KernelDesc>& kernels) {
  std::ostringstream o;
  o << kMagic << "\n";
  o << "// precompiled sm_100a entry points selected by name and element type; no source is compiled\n";
  for (auto& k : kernels) {
    o << "kernel " << kernel_entry_name(k.id) << "\n";
    o << "  element " << elt_name(k.elt) << "\n";
    o << "  block_m " << k.block_m << "\n  block_n " << k.block_n << "\n  block_k " << k.block_k
      << "\n  head_dim " << k.head_dim << "\n  threads " << k.threads << "\n  causal " << k.causal
      << "\n";
    for (auto& a : k.args) {
      o << "  arg " << a.index << " " << (a.is_pointer ? "pointer" : "scalar") << " " << a.dtype
        << " " << (int)a.role << " " << (a.name.empty() ? "_" : a.name) << "\n";
    }
    o << "end\n";
  }
  return o.str();
}

bool parse_descriptor(const std::string& text, std::vector<KernelDesc>& out, std::string& error) {
  out.clear();
  if (text.compare(0, std::strlen(kMagic), kMagic) != 0) {
    error = "metal error: MSL compilation failed: the source is not a tmcuda kernel descriptor "
            "(libtmcuda holds precompiled sm_100a kernels; pass the text tm_emit_msl returned)";
    return false;
  }
  std::istringstream in(text);
  std::string line;
  KernelDesc cur;
  bool open = false;
  auto bad = [&](const std::string& l) {
    error = "metal error: MSL compilation failed: malformed descriptor line '" + l + "'";
    return false;
  };
  while (std::getline(in, line)) {
    std::string t = trim(line);
    if (t.empty() || t.rfind("//", 0) == 0) continue;
    std::istringstream ls(t);
    std::string key;
    ls >> key;
    if (key == "kernel") {
      std::string name;
      ls >> name;
      cur = KernelDesc();
      bool known = false;
      for (int i = 0; i < (int)KernelId::Count; ++i)
        if (name == kernel_entry_name((KernelId)i)) { cur.id = (KernelId)i; known = true; }
      if (!known) return bad(t);
      open = true;
    } else if (!open) {
      return bad(t);
    } else if (key == "element") {
      std::string e;
      ls >> e;
      if (e == "f32") cur.elt = Elt::F32;
      else if (e == "f16") cur.elt = Elt::F16;
      else if (e == "bf16") cur.elt = Elt::BF16;
      else return bad(t);
    } else if (key == "block_m") { ls >> cur.block_m; }
    else if (key == "block_n") { ls >> cur.block_n; }
    else if (key == "block_k") { ls >> cur.block_k; }
    else if (key == "head_dim") { ls >> cur.head_dim; }
    else if (key == "threads") { ls >> cur.threads; }
    else if (key == "causal") { ls >> cur.causal; }
    else if (key == "arg") {
      ArgInfo a;
      std::string kind;
      int role = 0;
      ls >> a.index >> kind >> a.dtype >> role >> a.name;
      if (ls.fail() || (kind != "pointer" && kind != "scalar") || role < 0 || role > (int)Role::Last)
        return bad(t);
      a.is_pointer = kind == "pointer";
      a.role = (Role)role;
      if (a.index != (int)cur.args.size()) return bad(t);
      cur.args.push_back(a);
    } else if (key == "end") {
      // the same checks the IR scan applies: roles, their kinds, the element type of the entry
      std::string why;
      if (!check_roles(cur, why)) {
        error = "metal error: MSL compilation failed: descriptor of " +
                std::string(kernel_entry_name(cur.id)) + " is not usable: " + why;
        return false;
      }
      if ((is_rowwise(cur.id) || cur.id == KernelId::SaeEncode) && cur.elt != Elt::F32) {
        error = "metal error: MSL compilation failed: " + std::string(kernel_entry_name(cur.id)) +
                " is precompiled for f32 only";
        return false;
      }
      for (auto& a : cur.args) {
        const bool data_ptr = a.is_pointer && a.role != Role::L && a.role != Role::Delta;
        if (data_ptr && a.dtype != elt_name(cur.elt)) {
          error = "metal error: MSL compilation failed: descriptor of " +
                  std::string(kernel_entry_name(cur.id)) + " mixes element types";
          return false;
        }
      }
      out.push_back(cur);
      open = false;
    } else {
      return bad(t);
    }
    if (ls.fail()) return bad(t);
  }
  if (open || out.empty()) {
    error = "metal error: MSL compilation failed: descriptor holds no complete kernel";
    return false;
  }
  return true;
}

std::string kernel_info_json(const std::vector<KernelDesc>& kernels) {
  // Same keys, sorted, as EmissionResult.kernelInfoJSON (Compiler.swift:146-170).
  std::ostringstream o;
  o << "{\n  \"kernels\" : [\n";
  for (size_t i = 0; i < kernels.size(); ++i) {
    auto& k = kernels[i];
    std::vector<int> shape;
    switch (k.id) {
      case KernelId::Matmul: case KernelId::SaeEncode: shape = {k.block_m, k.block_n}; break;
      case KernelId::AttnBwdPreprocess: shape = {k.block_m, k.head_dim}; break;
      case KernelId::AttnBwdDkdv: shape = {k.block_n, k.block_m}; break;
      case KernelId::VecCopy: case KernelId::VecAdd: case KernelId::VecMul: case KernelId::ScaleBias:
      case KernelId::Softmax:
        shape = {k.block_m};
        break;
      default: shape = {k.block_m, k.block_n}; break;
    }
    long long size = 1;
    for (int s : shape) size *= (s > 0 ? s : 1);
    o << "    {\n      \"args\" : [\n";
    for (size_t j = 0; j < k.args.size(); ++j) {
      auto& a = k.args[j];
      o << "        {\n          \"dtype\" : \"" << a.dtype << "\",\n          \"index\" : " << a.index
        << ",\n          \"kind\" : \"" << (a.is_pointer ? "pointer" : "scalar") << "\"\n        }"
        << (j + 1 < k.args.size() ? "," : "") << "\n";
    }
    o << "      ],\n      \"block_shape\" : [";
    for (size_t j = 0; j < shape.size(); ++j) o << (j ? ", " : "") << shape[j];
    o << "],\n      \"block_size\" : " << size << ",\n      \"name\" : \"" << kernel_entry_name(k.id)
      << "\",\n      \"threads_per_threadgroup\" : " << k.threads << "\n    }"
      << (i + 1 < kernels.size() ? "," : "") << "\n";
  }
  o << "  ]\n}";
  return o.str();
}

}  // namespace tmc
