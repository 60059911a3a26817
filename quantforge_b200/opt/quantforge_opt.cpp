// quantforge-opt, re-hosted without MLIR: a small driver that reads the subset of MLIR text the
// W4A16 hot path uses and applies the hot-path passes under the reference's own flag names, plus
// the new pass that turns the matched ops into calls into the B200 runtime.
//
//   quantforge-opt [--convert-linalg-to-quantforge] [--fuse-unpack-dequant]
//                  [--canonicalize-dequant-zp] [--lower-qf-to-runtime]
//                  [-pass-pipeline='builtin.module(func.func(convert-linalg-to-quantforge{qf-bitwidth=4}))']
//                  [-o out.mlir] [file.mlir | -]
//
// Reference counterparts (paths inside the reference project):
//   driver                          tools/quantforge-opt/quantforge-opt.cpp:27-54
//   --convert-linalg-to-quantforge  lib/Transforms/ConvertLinalgToQuantForge.cpp:63-209 (option qf-bitwidth :223-225)
//   --fuse-unpack-dequant           lib/Transforms/FuseUnpackDequant.cpp:68-206 (same-shape form)
//   --canonicalize-dequant-zp       lib/Transforms/CanonicalizeDequantZeroPoint.cpp:103-197
//   --lower-qf-to-runtime           new: no counterpart; replaces matmul(x, qf.dequant(qf.unpack(w), s, z)) by
//                                   func.call @qf_w4a16_linear, a lone qf.unpack by @qf_unpack_int4 and a lone
//                                   qf.dequant(qf.unpack) by @qf_dequant_w4 (entry points of quantforge_rt.h).
// Exit code 0 on success, 1 on failure (diagnostics on stderr), as MlirOptMain's asMainReturnCode.
//   --lower-unpack-to-arith / --lower-unpack-branch-free / --lower-unpack-to-nvvm / --lower-unpack-to-prmt,
//   --lower-dequant-to-arith, --fuse-unpack-dequant-branch-free: the reference's scalar lowerings
//                                   (lib/Transforms/LowerUnpack*.cpp, LowerDequantToArith.cpp), emitted as text
// The reference's generic GPU scaffolding passes (tiling .. lower-to-nvvm) and register-layout-aware-unpack are
// not part of this build: asking for them is an error.
//
// The IR model is deliberately small: a module is a list of top-level chunks; a function is a header,
// a list of statements and a closing brace; a statement is the text of one operation (possibly spanning
// lines) with its result names and operation name extracted. Passes rewrite statements.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <regex>
#include <set>
#include <sstream>
#include <string>
#include <vector>

namespace {

struct Stmt {
    std::string text;      // full text, no trailing newline, original indentation kept
    std::string result;    // "%name" or ""
    std::string op;        // e.g. "linalg.matmul", "return"
};

struct Func {
    std::string header;            // "func.func @f(...) -> ... {"
    std::vector<Stmt> body;
    std::string footer = "}";
};

struct Chunk {
    bool is_func = false;
    std::string text;  // verbatim text for non-function chunks
    Func func;
};

struct Module {
    std::vector<Chunk> chunks;
    std::set<std::string> runtime_decls;  // private declarations to append
    std::vector<std::pair<std::string, std::string>> aliases;  // (#name, affine_map<...>) printed at the top
    // Attribute alias for an affine map, created on first use (#map, #map1, ...), as the MLIR printer hoists them.
    std::string alias(const std::string &map) {
        for (const auto &a : aliases)
            if (a.second == map) return a.first;
        const std::string name = aliases.empty() ? "#map" : "#map" + std::to_string(aliases.size());
        aliases.emplace_back(name, map);
        return name;
    }
};

[[noreturn]] void die(const std::string &msg) {
    std::cerr << "quantforge-opt: error: " << msg << "\n";
    std::exit(1);
}

std::string trim(const std::string &s) {
    size_t a = s.find_first_not_of(" \t\r\n");
    if (a == std::string::npos) return "";
    size_t b = s.find_last_not_of(" \t\r\n");
    return s.substr(a, b - a + 1);
}

// Depth of (), [], {}, <> nesting change of a line, ignoring "->" arrows and comments.
int depth_delta(const std::string &line) {
    int d = 0;
    for (size_t i = 0; i < line.size(); ++i) {
        char c = line[i];
        if (c == '/' && i + 1 < line.size() && line[i + 1] == '/') break;
        if (c == '-' && i + 1 < line.size() && line[i + 1] == '>') {
            ++i;
            continue;
        }
        if (c == '(' || c == '[' || c == '{' || c == '<') ++d;
        if (c == ')' || c == ']' || c == '}' || c == '>') --d;
    }
    return d;
}

std::string strip_comment(const std::string &line) {
    size_t p = line.find("//");
    return p == std::string::npos ? line : line.substr(0, p);
}

void classify(Stmt &s) {
    static const std::regex re_res(R"(^\s*(%[\w.\-#:]+)\s*=\s*([\w.]+))");
    static const std::regex re_op(R"(^\s*([\w.]+))");
    std::smatch m;
    if (std::regex_search(s.text, m, re_res)) {
        s.result = m[1];
        s.op = m[2];
    } else if (std::regex_search(s.text, m, re_op)) {
        s.op = m[1];
    }
}

Module parse(std::istream &in) {
    Module mod;
    // Comments are dropped on input, as the MLIR printer never reproduces them.
    std::vector<std::string> lines;
    for (std::string l; std::getline(in, l);) {
        std::string code = strip_comment(l);
        size_t e = code.find_last_not_of(" \t\r");
        code = e == std::string::npos ? "" : code.substr(0, e + 1);
        if (!code.empty()) lines.push_back(code);
    }
    size_t i = 0;
    std::string pending;
    auto flush_pending = [&]() {
        if (!pending.empty()) {
            Chunk c;
            c.text = pending;
            mod.chunks.push_back(c);
            pending.clear();
        }
    };
    while (i < lines.size()) {
        const std::string code = trim(strip_comment(lines[i]));
        if (code.rfind("func.func", 0) == 0) {
            flush_pending();
            Chunk c;
            c.is_func = true;
            // header: up to the line whose code ends with '{' at nesting depth 1
            std::string header;
            int depth = 0;
            bool declaration_only = false;
            while (i < lines.size()) {
                header += (header.empty() ? "" : "\n") + lines[i];
                depth += depth_delta(lines[i]);
                const std::string t = trim(strip_comment(lines[i]));
                ++i;
                if (!t.empty() && t.back() == '{' && depth == 1) break;
                if (depth == 0 && !t.empty() && t.back() != ',' && t.find("->") != std::string::npos &&
                    (i >= lines.size() || trim(strip_comment(lines[i])).rfind("{", 0) != 0)) {
                    declaration_only = (t.back() != '{');
                    if (declaration_only) break;
                }
            }
            if (declaration_only) {  // e.g. "func.func private @f(...) -> i32"
                Chunk d;
                d.text = header;
                mod.chunks.push_back(d);
                continue;
            }
            c.func.header = header;
            // body statements until the closing brace at depth 0
            depth = 1;
            std::string cur;
            int sdepth = 0;
            while (i < lines.size()) {
                const std::string t = trim(strip_comment(lines[i]));
                if (cur.empty() && t == "}") {
                    ++i;
                    depth = 0;
                    break;
                }
                if (cur.empty() && t.empty()) {  // blank or comment-only line inside a function: drop
                    ++i;
                    continue;
                }
                cur += (cur.empty() ? "" : "\n") + lines[i];
                sdepth += depth_delta(lines[i]);
                ++i;
                // a statement ends when brackets balance and the next line does not continue it
                bool cont = sdepth > 0;
                if (!cont && i < lines.size()) {
                    const std::string nt = trim(strip_comment(lines[i]));
                    if (nt.rfind("ins(", 0) == 0 || nt.rfind("outs(", 0) == 0 || nt.rfind("->", 0) == 0 ||
                        nt.rfind(":", 0) == 0 || (!t.empty() && (t.back() == ':' || t.back() == ',')))
                        cont = true;
                }
                if (!cont) {
                    Stmt s;
                    s.text = cur;
                    classify(s);
                    c.func.body.push_back(s);
                    cur.clear();
                    sdepth = 0;
                }
            }
            if (depth != 0) die("unterminated function body");
            mod.chunks.push_back(c);
        } else {
            pending += (pending.empty() ? "" : "\n") + lines[i];
            ++i;
        }
    }
    flush_pending();
    return mod;
}

void print(const Module &mod, std::ostream &os) {
    for (const auto &a : mod.aliases) os << a.first << " = " << a.second << "\n";
    bool wrote_decls = mod.runtime_decls.empty();
    for (const auto &c : mod.chunks) {
        if (!c.is_func) {
            if (trim(c.text).empty()) continue;
            os << c.text << "\n";
            continue;
        }
        if (!wrote_decls) {
            for (const auto &d : mod.runtime_decls) os << d << "\n";
            wrote_decls = true;
        }
        os << c.func.header << "\n";
        for (const auto &s : c.func.body) os << s.text << "\n";
        os << c.func.footer << "\n";
    }
    if (!wrote_decls)
        for (const auto &d : mod.runtime_decls) os << d << "\n";
}

// ---- small helpers on statement text -------------------------------------------------------------
std::string flat(const std::string &s) {  // collapse whitespace/newlines
    std::string o;
    bool sp = false;
    for (char c : s) {
        if (c == '\n' || c == '\t' || c == ' ' || c == '\r') {
            sp = true;
        } else {
            if (sp && !o.empty()) o += ' ';
            sp = false;
            o += c;
        }
    }
    return o;
}

struct TensorTy {
    std::vector<std::string> dims;
    std::string elem;
    bool ok = false;
    std::string str() const {
        std::string s = "tensor<";
        for (auto &d : dims) s += d + "x";
        return s + elem + ">";
    }
    TensorTy with_elem(const std::string &e) const {
        TensorTy t = *this;
        t.elem = e;
        return t;
    }
};

TensorTy parse_tensor(const std::string &t) {
    TensorTy r;
    static const std::regex re(R"(tensor<((?:[0-9?]+x)*)([a-z][a-z0-9]*)>)");
    std::smatch m;
    if (!std::regex_search(t, m, re)) return r;
    std::string dims = m[1];
    size_t p = 0;
    while (p < dims.size()) {
        size_t q = dims.find('x', p);
        r.dims.push_back(dims.substr(p, q - p));
        p = q + 1;
    }
    r.elem = m[2];
    r.ok = true;
    return r;
}

std::string indent_of(const std::string &text) {
    size_t a = text.find_first_not_of(" \t");
    return a == std::string::npos ? "" : text.substr(0, a);
}

int g_fresh = 0;
std::string fresh(const std::string &base) { return "%" + base + "_qf" + std::to_string(g_fresh++); }

const Stmt *find_def(const Func &f, const std::string &name) {
    for (const auto &s : f.body)
        if (s.result == name) return &s;
    return nullptr;
}

bool is_used_elsewhere(const Func &f, const std::string &name, const Stmt *except) {
    const std::regex re(name.substr(0, 1) == "%" ? "\\" + name + R"((?![\w.\-#]))" : name);
    for (const auto &s : f.body) {
        if (&s == except) continue;
        std::string t = s.text;
        if (s.result == name) {  // skip the definition's own LHS
            size_t eq = t.find('=');
            t = t.substr(eq + 1);
        }
        if (std::regex_search(t, re)) return true;
    }
    return false;
}

// Parsed linalg.matmul
struct Matmul {
    std::string attrs;  // "{...}" or ""
    std::string lhs, rhs, init;
    TensorTy lhs_ty, rhs_ty, init_ty, res_ty;
    bool ok = false;
};

Matmul parse_matmul(const Stmt &s) {
    Matmul m;
    const std::string t = flat(s.text);
    static const std::regex re(
        R"(linalg\.matmul\s*(\{.*\})?\s*ins\(\s*(%[\w.\-#]+)\s*,\s*(%[\w.\-#]+)\s*:\s*(tensor<[^>]*>)\s*,\s*(tensor<[^>]*>)\s*\)\s*outs\(\s*(%[\w.\-#]+)\s*:\s*(tensor<[^>]*>)\s*\)\s*->\s*(tensor<[^>]*>))");
    std::smatch r;
    if (!std::regex_search(t, r, re)) return m;
    m.attrs = r[1];
    m.lhs = r[2];
    m.rhs = r[3];
    m.lhs_ty = parse_tensor(r[4]);
    m.rhs_ty = parse_tensor(r[5]);
    m.init = r[6];
    m.init_ty = parse_tensor(r[7]);
    m.res_ty = parse_tensor(r[8]);
    m.ok = m.lhs_ty.ok && m.rhs_ty.ok && m.init_ty.ok && m.res_ty.ok;
    return m;
}

// "qf.scale = dense<...> : tensor<f16>" inside an attribute dictionary -> "dense<...>"
std::string harvest_attr(const std::string &text, const std::string &key) {
    const std::regex re(key + R"(\s*=\s*(dense<[^>]*>)\s*:\s*tensor<[a-z0-9]+>)");
    std::smatch m;
    const std::string t = flat(text);
    if (std::regex_search(t, m, re)) return m[1];
    return "";
}

struct Dequant {
    std::string in, scale, zp, attrs;
    TensorTy in_ty, out_ty;
    std::string scale_ty, zp_ty;
    bool ok = false;
};

Dequant parse_dequant(const Stmt &s) {
    Dequant d;
    const std::string t = flat(s.text);
    static const std::regex re(
        R"(qf\.dequant\s*(%[\w.\-#]+)\s*,\s*(%[\w.\-#]+)\s*,\s*(%[\w.\-#]+)\s*(\{.*\})?\s*:\s*(tensor<[^>]*>)\s*,\s*(tensor<[^>]*>)\s*,\s*(tensor<[^>]*>)\s*->\s*(tensor<[^>]*>))");
    std::smatch r;
    if (!std::regex_search(t, r, re)) return d;
    d.in = r[1];
    d.scale = r[2];
    d.zp = r[3];
    d.attrs = r[4];
    d.in_ty = parse_tensor(r[5]);
    d.scale_ty = r[6];
    d.zp_ty = r[7];
    d.out_ty = parse_tensor(r[8]);
    d.ok = d.in_ty.ok && d.out_ty.ok;
    return d;
}

struct Unpack {
    std::string in, attrs;
    TensorTy in_ty, out_ty;
    bool ok = false;
};

Unpack parse_unpack(const Stmt &s) {
    Unpack u;
    const std::string t = flat(s.text);
    static const std::regex re(R"(qf\.unpack\s*(%[\w.\-#]+)\s*(\{.*\})?\s*:\s*(tensor<[^>]*>)\s*->\s*(tensor<[^>]*>))");
    std::smatch r;
    if (!std::regex_search(t, r, re)) return u;
    u.in = r[1];
    u.attrs = r[2];
    u.in_ty = parse_tensor(r[3]);
    u.out_ty = parse_tensor(r[4]);
    u.ok = u.in_ty.ok && u.out_ty.ok;
    return u;
}

Stmt mk(const std::string &text) {
    Stmt s;
    s.text = text;
    classify(s);
    return s;
}

std::string identity_map(size_t rank) {
    std::string d;
    for (size_t i = 0; i < rank; ++i) d += (i ? ", d" : "d") + std::to_string(i);
    return "affine_map<(" + d + ") -> (" + d + ")>";
}
std::string scalar_map(size_t rank) {
    std::string d;
    for (size_t i = 0; i < rank; ++i) d += (i ? ", d" : "d") + std::to_string(i);
    return "affine_map<(" + d + ") -> ()>";
}
std::string iter_types(size_t rank) {
    std::string s;
    for (size_t i = 0; i < rank; ++i) s += (i ? ", \"parallel\"" : "\"parallel\"");
    return "[" + s + "]";
}

// ---- pass: convert-linalg-to-quantforge -----------------------------------------------------------
// linalg.matmul whose RHS is a rank-2 i8 tensor -> qf.unpack (same shape) + qf.dequant (scale / zero point from
// qf.scale / qf.zp attributes on the matmul or on the op defining the weight, else 1.0 / 0) + f16 matmul.
void pass_convert(Module &mod, int bitwidth) {
    if (bitwidth != 8 && bitwidth != 4) die("convert-linalg-to-quantforge: qf-bitwidth must be 4 or 8");
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::vector<Stmt> out;
        for (size_t i = 0; i < f.body.size(); ++i) {
            const Stmt &s = f.body[i];
            Matmul m;
            if (s.op == "linalg.matmul") m = parse_matmul(s);
            if (!m.ok || m.rhs_ty.elem != "i8" || m.rhs_ty.dims.size() != 2) {
                out.push_back(s);
                continue;
            }
            const std::string ind = indent_of(s.text);
            std::string scale = harvest_attr(m.attrs, "qf\\.scale");
            std::string zp = harvest_attr(m.attrs, "qf\\.zp");
            if (const Stmt *def = find_def(f, m.rhs)) {
                if (scale.empty()) scale = harvest_attr(def->text, "qf\\.scale");
                if (zp.empty()) zp = harvest_attr(def->text, "qf\\.zp");
            }
            if (scale.empty()) scale = "dense<1.000000e+00>";
            if (zp.empty()) zp = "dense<0>";
            const TensorTy w_i8 = m.rhs_ty;
            const TensorTy w_f16 = m.rhs_ty.with_elem("f16");
            const std::string u = fresh("unpack"), sc = fresh("scale"), z = fresh("zp"), dq = fresh("dequant");
            // Where the weight itself is a constant of the function, MLIR's folder keeps the new constants with it,
            // ahead of the unpack (the order the reference's tests with attribute-carrying constants expect).
            const Stmt *wdef = find_def(f, m.rhs);
            const bool consts_first = wdef && wdef->op == "arith.constant";
            if (!consts_first)
                out.push_back(mk(ind + u + " = qf.unpack " + m.rhs + " : " + w_i8.str() + " -> " + w_i8.str()));
            out.push_back(mk(ind + sc + " = arith.constant " + scale + " : tensor<f16>"));
            out.push_back(mk(ind + z + " = arith.constant " + zp + " : tensor<i8>"));
            if (consts_first)
                out.push_back(mk(ind + u + " = qf.unpack " + m.rhs + " : " + w_i8.str() + " -> " + w_i8.str()));
            out.push_back(mk(ind + dq + " = qf.dequant " + u + ", " + sc + ", " + z + " : " + w_i8.str() +
                             ", tensor<f16>, tensor<i8> -> " + w_f16.str()));
            std::string lhs = m.lhs;
            TensorTy lhs_ty = m.lhs_ty;
            if (lhs_ty.elem != "f16") {
                const std::string cast = fresh("lhs");
                out.push_back(mk(ind + cast + " = arith.sitofp " + lhs + " : " + lhs_ty.str() + " to " +
                                 lhs_ty.with_elem("f16").str()));
                lhs = cast;
                lhs_ty = lhs_ty.with_elem("f16");
            }
            const TensorTy init_ty = m.init_ty.with_elem("f16");
            const std::string e = fresh("empty"), zero = fresh("zero"), fill = fresh("fill");
            out.push_back(mk(ind + e + " = tensor.empty() : " + init_ty.str()));
            out.push_back(mk(ind + zero + " = arith.constant 0.000000e+00 : f16"));
            out.push_back(mk(ind + fill + " = linalg.fill ins(" + zero + " : f16) outs(" + e + " : " + init_ty.str() +
                             ") -> " + init_ty.str()));
            out.push_back(mk(ind + s.result + " = linalg.matmul ins(" + lhs + ", " + dq + " : " + lhs_ty.str() + ", " +
                             w_f16.str() + ") outs(" + fill + " : " + init_ty.str() + ") -> " + init_ty.str()));
        }
        f.body.swap(out);
    }
}

// ---- pass: fuse-unpack-dequant / canonicalize-dequant-zp ------------------------------------------------
std::string generic_dequant(const std::string &ind, const std::string &result, const std::string &in,
                            const Dequant &d, bool mask_nibble, bool with_zp, std::vector<Stmt> &out) {
    const size_t rank = d.out_ty.dims.size();
    const std::string e = fresh("empty");
    out.push_back(mk(ind + e + " = tensor.empty() : " + d.out_ty.str()));
    std::string t;
    if (with_zp) {
        t = ind + result + " = linalg.generic {indexing_maps = [" + identity_map(rank) + ", " + scalar_map(rank) + ", " +
            scalar_map(rank) + ", " + identity_map(rank) + "], iterator_types = " + iter_types(rank) + "} ins(" + in +
            ", " + d.scale + ", " + d.zp + " : " + d.in_ty.str() + ", " + d.scale_ty + ", " + d.zp_ty + ") outs(" + e +
            " : " + d.out_ty.str() + ") {\n";
        t += ind + "^bb0(%in: i8, %s: f16, %z: i8, %out: f16):\n";
    } else {
        t = ind + result + " = linalg.generic {indexing_maps = [" + identity_map(rank) + ", " + scalar_map(rank) + ", " +
            identity_map(rank) + "], iterator_types = " + iter_types(rank) + "} ins(" + in + ", " + d.scale + " : " +
            d.in_ty.str() + ", " + d.scale_ty + ") outs(" + e + " : " + d.out_ty.str() + ") {\n";
        t += ind + "^bb0(%in: i8, %s: f16, %out: f16):\n";
    }
    std::string v = "%in";
    if (mask_nibble) {
        t += ind + "  %c15 = arith.constant 15 : i8\n";
        t += ind + "  %m = arith.andi %in, %c15 : i8\n";
        v = "%m";
    }
    t += ind + "  %f = arith.sitofp " + v + " : i8 to f16\n";
    if (with_zp) {
        t += ind + "  %zf = arith.sitofp %z : i8 to f16\n";
        t += ind + "  %d = arith.subf %f, %zf : f16\n";
        t += ind + "  %r = arith.mulf %d, %s : f16\n";
    } else {
        t += ind + "  %r = arith.mulf %f, %s : f16\n";
    }
    t += ind + "  linalg.yield %r : f16\n";
    t += ind + "} -> " + d.out_ty.str();
    out.push_back(mk(t));
    return result;
}

// qf.dequant(qf.unpack(x)) with a same-shape unpack -> one pointwise linalg.generic (mask 0x0F + dequant).
void pass_fuse(Module &mod) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::set<std::string> dead_unpacks;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            if (s.op != "qf.dequant") {
                out.push_back(s);
                continue;
            }
            Dequant d = parse_dequant(s);
            const Stmt *def = d.ok ? find_def(f, d.in) : nullptr;
            Unpack u;
            if (def && def->op == "qf.unpack") u = parse_unpack(*def);
            if (!u.ok || d.out_ty.elem != "f16") {
                out.push_back(s);
                continue;
            }
            if (u.in_ty.dims != u.out_ty.dims) {
                // shape-doubling form: [.., n] packed -> [.., n, 2] generic (nibble select by the innermost index) -> collapse
                const size_t r = u.in_ty.dims.size();
                bool doubles = r >= 1 && u.out_ty.dims.size() == r;
                for (size_t k = 0; doubles && k + 1 < r; ++k) doubles = u.in_ty.dims[k] == u.out_ty.dims[k];
                if (doubles) doubles = std::to_string(2 * std::stoll(u.in_ty.dims[r - 1])) == u.out_ty.dims[r - 1];
                if (!doubles) {
                    out.push_back(s);
                    continue;
                }
                const std::string ind = indent_of(s.text);
                TensorTy wide = u.in_ty.with_elem("f16");
                wide.dims.push_back("2");
                const std::string c15 = fresh("c15"), c4 = fresh("c4"), c0 = fresh("c0"), e = fresh("empty"), gen = fresh("fused");
                out.push_back(mk(ind + c15 + " = arith.constant 15 : i8"));
                out.push_back(mk(ind + c4 + " = arith.constant 4 : i8"));
                out.push_back(mk(ind + c0 + " = arith.constant 0 : index"));
                out.push_back(mk(ind + e + " = tensor.empty() : " + wide.str()));
                std::string dims, lhs_dims;
                for (size_t k = 0; k <= r; ++k) dims += (k ? ", d" : "d") + std::to_string(k);
                for (size_t k = 0; k < r; ++k) lhs_dims += (k ? ", d" : "d") + std::to_string(k);
                const std::string in_map = "affine_map<(" + dims + ") -> (" + lhs_dims + ")>";
                std::string t = ind + gen + " = linalg.generic {indexing_maps = [" + in_map + ", " + scalar_map(r + 1) + ", " +
                                scalar_map(r + 1) + ", " + identity_map(r + 1) + "], iterator_types = " + iter_types(r + 1) +
                                "} ins(" + u.in + ", " + d.scale + ", " + d.zp + " : " + u.in_ty.str() + ", " + d.scale_ty +
                                ", " + d.zp_ty + ") outs(" + e + " : " + wide.str() + ") {\n";
                t += ind + "^bb0(%in: i8, %s: f16, %z: i8, %out: f16):\n";
                t += ind + "  %lo = arith.andi %in, " + c15 + " : i8\n";
                t += ind + "  %sh = arith.shrui %in, " + c4 + " : i8\n";
                t += ind + "  %hi = arith.andi %sh, " + c15 + " : i8\n";
                t += ind + "  %idx = linalg.index " + std::to_string(r) + " : index\n";
                t += ind + "  %is_lo = arith.cmpi eq, %idx, " + c0 + " : index\n";
                t += ind + "  %q = arith.select %is_lo, %lo, %hi : i8\n";
                t += ind + "  %f = arith.sitofp %q : i8 to f16\n";
                t += ind + "  %zf = arith.sitofp %z : i8 to f16\n";
                t += ind + "  %d = arith.subf %f, %zf : f16\n";
                t += ind + "  %r = arith.mulf %d, %s : f16\n";
                t += ind + "  linalg.yield %r : f16\n";
                t += ind + "} -> " + wide.str();
                out.push_back(mk(t));
                std::string reassoc = "[";
                for (size_t k = 0; k + 1 < r; ++k) reassoc += "[" + std::to_string(k) + "], ";
                reassoc += "[" + std::to_string(r - 1) + ", " + std::to_string(r) + "]]";
                out.push_back(mk(ind + s.result + " = tensor.collapse_shape " + gen + " " + reassoc + " : " + wide.str() +
                                 " into " + d.out_ty.str()));
                dead_unpacks.insert(def->result);
                continue;
            }
            Dequant dd = d;
            dd.in_ty = u.in_ty;
            generic_dequant(indent_of(s.text), s.result, u.in, dd, /*mask*/ true, /*zp*/ true, out);
            dead_unpacks.insert(def->result);
        }
        f.body.swap(out);
        // drop unpacks that lost their only user
        std::vector<Stmt> kept;
        for (const Stmt &s : f.body) {
            if (s.op == "qf.unpack" && dead_unpacks.count(s.result) && !is_used_elsewhere(f, s.result, &s)) continue;
            kept.push_back(s);
        }
        f.body.swap(kept);
    }
}

bool is_zero_constant(const Func &f, const std::string &name) {
    const Stmt *def = find_def(f, name);
    if (!def || def->op != "arith.constant") return false;
    static const std::regex re(R"(arith\.constant\s+dense<\s*0\s*>\s*:\s*tensor<i8>)");
    return std::regex_search(flat(def->text), re);
}

// qf.dequant whose zero point is the constant 0 -> generic with sitofp + mulf only.
void pass_canonicalize_zp(Module &mod) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            Dequant d;
            if (s.op == "qf.dequant") d = parse_dequant(s);
            if (!d.ok || !is_zero_constant(f, d.zp) || d.out_ty.elem != "f16") {
                out.push_back(s);
                continue;
            }
            generic_dequant(indent_of(s.text), s.result, d.in, d, /*mask*/ false, /*zp*/ false, out);
        }
        f.body.swap(out);
        // arith.subf %x, <constant 0.0>  ->  %x   (lib/Transforms/CanonicalizeDequantZeroPoint.cpp:207-230)
        {
            static const std::regex re_sub(R"(arith\.subf\s+(%[\w.\-#]+)\s*,\s*(%[\w.\-#]+)\s*:)");
            static const std::regex re_zero(R"(arith\.constant\s+0(\.0+(e[+-]?0+)?)?\s*:\s*(f16|f32|bf16))");
            std::vector<Stmt> body2;
            std::map<std::string, std::string> repl;
            for (Stmt s : f.body) {
                for (const auto &kv : repl)
                    s.text = std::regex_replace(s.text, std::regex("\\" + kv.first + R"((?![\w.\-#]))"), kv.second);
                std::smatch m;
                const std::string t = flat(s.text);
                if (s.op == "arith.subf" && std::regex_search(t, m, re_sub)) {
                    const Stmt *zdef = find_def(f, m[2]);
                    if (zdef && zdef->op == "arith.constant" && std::regex_search(flat(zdef->text), re_zero)) {
                        repl[s.result] = m[1];
                        continue;
                    }
                }
                body2.push_back(s);
            }
            f.body.swap(body2);
            std::vector<Stmt> body3;  // float zero constants that lost their last user
            for (const Stmt &s : f.body) {
                if (s.op == "arith.constant" && std::regex_search(flat(s.text), re_zero) && !repl.empty() &&
                    !is_used_elsewhere(f, s.result, &s))
                    continue;
                body3.push_back(s);
            }
            f.body.swap(body3);
        }
        std::vector<Stmt> kept;  // dead zero constants
        for (const Stmt &s : f.body) {
            if (s.op == "arith.constant" && is_zero_constant(f, s.result) && !is_used_elsewhere(f, s.result, &s)) continue;
            kept.push_back(s);
        }
        f.body.swap(kept);
    }
}

// ---- pass: lower-qf-to-runtime -----------------------------------------------------------------------
// Attributes carried from the dequant op's attr-dict (group_size, zero_mode, zero_const, out_dtype) onto the call.
std::string call_attrs(const Dequant &d, const std::string &extra) {
    std::string inner = d.attrs.size() >= 2 ? trim(d.attrs.substr(1, d.attrs.size() - 2)) : "";
    if (inner.find("group_size") == std::string::npos) inner += (inner.empty() ? "" : ", ") + std::string("group_size = 0 : i64");
    if (!extra.empty()) inner += ", " + extra;
    return " {" + inner + "}";
}

void pass_lower_to_runtime(Module &mod) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        // 1. matmul(x, dequant(unpack(w)))
        std::vector<Stmt> out;
        std::set<std::string> maybe_dead;
        for (const Stmt &s : f.body) {
            Matmul m;
            if (s.op == "linalg.matmul") m = parse_matmul(s);
            const Stmt *dq_def = m.ok ? find_def(f, m.rhs) : nullptr;
            Dequant d;
            if (dq_def && dq_def->op == "qf.dequant") d = parse_dequant(*dq_def);
            const Stmt *u_def = d.ok ? find_def(f, d.in) : nullptr;
            Unpack u;
            if (u_def && u_def->op == "qf.unpack") u = parse_unpack(*u_def);
            if (!u.ok || m.lhs_ty.dims.size() != 2 || m.rhs_ty.dims.size() != 2) {
                out.push_back(s);
                continue;
            }
            const std::string sig = "(" + m.lhs_ty.str() + ", " + u.in_ty.str() + ", " + d.scale_ty + ", " + d.zp_ty +
                                    ", " + m.init_ty.str() + ") -> " + m.res_ty.str();
            // weights in the IR are [K, N] (B operand of linalg.matmul); the runtime takes them [N, K/2]
            // one MLIR symbol per shape (MLIR has no overloading); all of them bind to the same C entry point
            const std::string sym = "@qf_w4a16_linear_m" + m.lhs_ty.dims[0] + "_k" + m.rhs_ty.dims[0] + "_n" + m.rhs_ty.dims[1];
            out.push_back(mk(indent_of(s.text) + s.result + " = func.call " + sym + "(" + m.lhs + ", " + u.in +
                             ", " + d.scale + ", " + d.zp + ", " + m.init + ")" +
                             call_attrs(d, "qf.weight_orientation = \"kn\"") + " : " + sig));
            mod.runtime_decls.insert("func.func private " + sym + sig +
                                     " attributes {qf.runtime_symbol = \"qf_w4a16_linear\"}");
            maybe_dead.insert(dq_def->result);
            maybe_dead.insert(u_def->result);
        }
        f.body.swap(out);
        auto sweep_dead = [&]() {
            bool changed = true;
            while (changed) {
                changed = false;
                std::vector<Stmt> kept;
                for (const Stmt &s : f.body) {
                    if (maybe_dead.count(s.result) && (s.op == "qf.dequant" || s.op == "qf.unpack") &&
                        !is_used_elsewhere(f, s.result, &s)) {
                        changed = true;
                        continue;
                    }
                    kept.push_back(s);
                }
                f.body.swap(kept);
            }
        };
        sweep_dead();
        // 2. remaining dequant(unpack(w)) -> qf_dequant_w4 ; remaining unpack -> qf_unpack_int4
        out.clear();
        for (const Stmt &s : f.body) {
            if (s.op == "qf.dequant") {
                Dequant d = parse_dequant(s);
                const Stmt *u_def = d.ok ? find_def(f, d.in) : nullptr;
                Unpack u;
                if (u_def && u_def->op == "qf.unpack") u = parse_unpack(*u_def);
                if (u.ok) {
                    const std::string sig = "(" + u.in_ty.str() + ", " + d.scale_ty + ", " + d.zp_ty + ") -> " + d.out_ty.str();
                    const std::string sym = "@qf_dequant_w4_" + u.in_ty.dims[0] + "x" + u.in_ty.dims[1];
                    out.push_back(mk(indent_of(s.text) + s.result + " = func.call " + sym + "(" + u.in + ", " +
                                     d.scale + ", " + d.zp + ")" + call_attrs(d, "") + " : " + sig));
                    mod.runtime_decls.insert("func.func private " + sym + sig +
                                             " attributes {qf.runtime_symbol = \"qf_dequant_w4\"}");
                    maybe_dead.insert(u_def->result);
                    continue;
                }
            }
            out.push_back(s);
        }
        f.body.swap(out);
        sweep_dead();
        out.clear();
        for (const Stmt &s : f.body) {
            if (s.op == "qf.unpack") {
                Unpack u = parse_unpack(s);
                if (u.ok) {
                    const std::string sig = "(" + u.in_ty.str() + ") -> " + u.out_ty.str();
                    const std::string sym = "@qf_unpack_int4_" + u.in_ty.dims[0] + "x" + u.in_ty.dims.back();
                    out.push_back(mk(indent_of(s.text) + s.result + " = func.call " + sym + "(" + u.in + ") : " + sig));
                    mod.runtime_decls.insert("func.func private " + sym + sig +
                                             " attributes {qf.runtime_symbol = \"qf_unpack_int4\"}");
                    continue;
                }
            }
            out.push_back(s);
        }
        f.body.swap(out);
        // 3. there is no CPU fallback: anything of the dialect that is left is an error
        for (const Stmt &s : f.body)
            if (s.op.rfind("qf.", 0) == 0)
                die("lower-qf-to-runtime: cannot lower '" + flat(s.text) + "' to a runtime call (no CPU fallback exists)");
    }
}


// ---- the reference's scalar lowerings of qf.unpack / qf.dequant ----------------------------------------
// They define the arithmetic the runtime kernels implement (and the CPU oracle restates); emitting them keeps the
// driver usable for inspecting that arithmetic and keeps every reference flag of the hot path alive.

// [.., n] -> [.., 2n] with every leading extent equal
bool unpack_doubles(const Unpack &u) {
    const size_t r = u.in_ty.dims.size();
    if (r < 1 || u.out_ty.dims.size() != r) return false;
    for (size_t k = 0; k + 1 < r; ++k)
        if (u.in_ty.dims[k] != u.out_ty.dims[k]) return false;
    for (const auto &d : u.in_ty.dims)
        if (d == "?") return false;
    return std::to_string(2 * std::stoll(u.in_ty.dims[r - 1])) == u.out_ty.dims[r - 1];
}

std::string dim_list(size_t n) {
    std::string d;
    for (size_t k = 0; k < n; ++k) d += (k ? ", d" : "d") + std::to_string(k);
    return d;
}

// --lower-unpack-to-arith (lib/Transforms/LowerUnpackToArith.cpp:73-219): one generic over [.., n, 2] that selects
// the low or the high nibble by the innermost index, then a collapse to [.., 2n].
void pass_lower_unpack_to_arith(Module &mod) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            Unpack u;
            if (s.op == "qf.unpack") u = parse_unpack(s);
            if (!u.ok || u.in_ty.elem != "i8" || !unpack_doubles(u)) {
                out.push_back(s);
                continue;
            }
            const size_t r = u.in_ty.dims.size();
            const std::string ind = indent_of(s.text);
            TensorTy wide = u.in_ty;
            wide.dims.push_back("2");
            const std::string in_map = mod.alias("affine_map<(" + dim_list(r + 1) + ") -> (" + dim_list(r) + ")>");
            const std::string out_map = mod.alias("affine_map<(" + dim_list(r + 1) + ") -> (" + dim_list(r + 1) + ")>");
            const std::string c15 = fresh("c15"), c4 = fresh("c4"), c0 = fresh("c0"), e = fresh("empty"), gen = fresh("unpacked");
            out.push_back(mk(ind + c15 + " = arith.constant 15 : i8"));
            out.push_back(mk(ind + c4 + " = arith.constant 4 : i8"));
            out.push_back(mk(ind + c0 + " = arith.constant 0 : index"));
            out.push_back(mk(ind + e + " = tensor.empty() : " + wide.str()));
            std::string t = ind + gen + " = linalg.generic {indexing_maps = [" + in_map + ", " + out_map +
                            "], iterator_types = " + iter_types(r + 1) + "} ins(" + u.in + " : " + u.in_ty.str() +
                            ") outs(" + e + " : " + wide.str() + ") {\n";
            t += ind + "^bb0(%in: i8, %out: i8):\n";
            t += ind + "  %lo = arith.andi %in, " + c15 + " : i8\n";
            t += ind + "  %sh = arith.shrui %in, " + c4 + " : i8\n";
            t += ind + "  %hi = arith.andi %sh, " + c15 + " : i8\n";
            t += ind + "  %idx = linalg.index " + std::to_string(r) + " : index\n";
            t += ind + "  %is_lo = arith.cmpi eq, %idx, " + c0 + " : index\n";
            t += ind + "  %q = arith.select %is_lo, %lo, %hi : i8\n";
            t += ind + "  linalg.yield %q : i8\n";
            t += ind + "} -> " + wide.str();
            out.push_back(mk(t));
            std::string reassoc = "[";
            for (size_t k = 0; k + 1 < r; ++k) reassoc += "[" + std::to_string(k) + "], ";
            reassoc += "[" + std::to_string(r - 1) + ", " + std::to_string(r) + "]]";
            out.push_back(mk(ind + s.result + " = tensor.collapse_shape " + gen + " " + reassoc + " : " + wide.str() +
                             " into " + u.out_ty.str()));
        }
        f.body.swap(out);
    }
}

// Pointwise generic over `ty` whose body is `lines` (each without indentation), yielding %r of element type `elem_out`.
std::string pointwise_generic(const std::string &ind, const std::string &result, const std::string &ins,
                              const std::string &ins_types, const std::string &maps, size_t rank,
                              const std::string &out_buf, const TensorTy &out_ty, const std::string &bb_args,
                              const std::vector<std::string> &lines) {
    std::string t = ind + result + " = linalg.generic {indexing_maps = [" + maps + "], iterator_types = " +
                    iter_types(rank) + "} ins(" + ins + " : " + ins_types + ") outs(" + out_buf + " : " + out_ty.str() +
                    ") {\n";
    t += ind + "^bb0(" + bb_args + "):\n";
    for (const auto &l : lines) t += ind + "  " + l + "\n";
    t += ind + "  linalg.yield %r : " + out_ty.elem + "\n";
    t += ind + "} -> " + out_ty.str();
    return t;
}

std::string slice_spec(const TensorTy &half, int offset_last) {
    std::string off = "[", size = "[", stride = "[";
    const size_t r = half.dims.size();
    for (size_t k = 0; k < r; ++k) {
        const bool last = k + 1 == r;
        off += std::string(k ? ", " : "") + (last ? std::to_string(offset_last) : "0");
        size += std::string(k ? ", " : "") + half.dims[k];
        stride += std::string(k ? ", " : "") + (last ? "2" : "1");
    }
    return off + "] " + size + "] " + stride + "]";
}

// --lower-unpack-branch-free (lib/Transforms/LowerUnpackBranchFree.cpp:78-230): low and high nibbles as two
// pointwise generics, interleaved by two stride-2 tensor.insert_slice: out[.., 2n] = low, out[.., 2n+1] = high.
// --fuse-unpack-dequant-branch-free (lib/Transforms/FuseUnpackDequant.cpp:323-508): the same with the dequant
// arithmetic inside both generics.
void pass_branch_free(Module &mod, bool fuse_dequant) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::set<std::string> dead_unpacks;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            Unpack u;
            Dequant d;
            const Stmt *def = nullptr;
            if (!fuse_dequant && s.op == "qf.unpack") {
                u = parse_unpack(s);
            } else if (fuse_dequant && s.op == "qf.dequant") {
                d = parse_dequant(s);
                def = d.ok ? find_def(f, d.in) : nullptr;
                if (def && def->op == "qf.unpack") u = parse_unpack(*def);
                if (d.ok && d.out_ty.elem != "f16") u.ok = false;
            }
            if (!u.ok || u.in_ty.elem != "i8" || !unpack_doubles(u)) {
                out.push_back(s);
                continue;
            }
            const size_t r = u.in_ty.dims.size();
            const std::string ind = indent_of(s.text);
            const std::string id = identity_map(r);
            const TensorTy half = fuse_dequant ? u.in_ty.with_elem("f16") : u.in_ty;
            const TensorTy full = fuse_dequant ? d.out_ty : u.out_ty;
            const std::string c15 = fresh("c15"), c4 = fresh("c4");
            out.push_back(mk(ind + c15 + " = arith.constant 15 : i8"));
            out.push_back(mk(ind + c4 + " = arith.constant 4 : i8"));
            std::string halves[2];
            for (int hi = 0; hi < 2; ++hi) {
                const std::string e = fresh("empty"), g = fresh(hi ? "high" : "low");
                out.push_back(mk(ind + e + " = tensor.empty() : " + half.str()));
                std::vector<std::string> body;
                std::string v = "%b";
                if (hi) {
                    body.push_back("%sh = arith.shrui %b, " + c4 + " : i8");
                    v = "%sh";
                }
                if (fuse_dequant) {
                    body.push_back("%m = arith.andi " + v + ", " + c15 + " : i8");
                    body.push_back("%qf = arith.sitofp %m : i8 to f16");
                    body.push_back("%zf = arith.sitofp %z : i8 to f16");
                    body.push_back("%d = arith.subf %qf, %zf : f16");
                    body.push_back("%r = arith.mulf %d, %s : f16");
                    out.push_back(mk(pointwise_generic(
                        ind, g, u.in + ", " + d.scale + ", " + d.zp, u.in_ty.str() + ", " + d.scale_ty + ", " + d.zp_ty,
                        id + ", " + scalar_map(r) + ", " + scalar_map(r) + ", " + id, r, e, half,
                        "%b: i8, %s: f16, %z: i8, %o: f16", body)));
                } else {
                    body.push_back("%r = arith.andi " + v + ", " + c15 + " : i8");
                    out.push_back(mk(pointwise_generic(ind, g, u.in, u.in_ty.str(), id + ", " + id, r, e, half,
                                                       "%b: i8, %o: i8", body)));
                }
                halves[hi] = g;
            }
            const std::string o = fresh("out"), i0 = fresh("interleaved");
            out.push_back(mk(ind + o + " = tensor.empty() : " + full.str()));
            out.push_back(mk(ind + i0 + " = tensor.insert_slice " + halves[0] + " into " + o + slice_spec(half, 0) + " : " +
                             half.str() + " into " + full.str()));
            out.push_back(mk(ind + s.result + " = tensor.insert_slice " + halves[1] + " into " + i0 + slice_spec(half, 1) +
                             " : " + half.str() + " into " + full.str()));
            if (def) dead_unpacks.insert(def->result);
        }
        f.body.swap(out);
        std::vector<Stmt> kept;
        for (const Stmt &s : f.body) {
            if (s.op == "qf.unpack" && dead_unpacks.count(s.result) && !is_used_elsewhere(f, s.result, &s)) continue;
            kept.push_back(s);
        }
        f.body.swap(kept);
    }
}

// --lower-unpack-to-nvvm (lib/Transforms/LowerUnpackToNVVM.cpp:90-295) and --lower-unpack-to-prmt
// (lib/Transforms/LowerUnpackToPRMT.cpp:293-350): scf.for over rows x 4-byte chunks; four bytes are read and
// joined into one i32 word, the eight codes leave it LSB first (code n = (w >> 4n) & 0xF) and are written with
// eight tensor.insert. Guards as in the reference: rank 2, static shape, doubling form, packed columns % 4 == 0.
// The prmt variant spreads the codes to one byte each with two prmt.b32 on the nibble-masked words
//   lo = w & 0x0F0F0F0F, hi = (w >> 4) & 0x0F0F0F0F, prmt(lo, hi, 0x5140) = codes 0..3, prmt(lo, hi, 0x7362) = 4..7
// which is what the runtime's unpack kernel executes (the reference names the same two selectors but applies them
// to the unmasked word with zero as second operand, which does not separate the nibbles on hardware).
void pass_lower_unpack_loops(Module &mod, bool use_prmt) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            Unpack u;
            if (s.op == "qf.unpack") u = parse_unpack(s);
            const bool ok = u.ok && u.in_ty.elem == "i8" && u.in_ty.dims.size() == 2 && unpack_doubles(u) &&
                            std::stoll(u.in_ty.dims[1]) % 4 == 0;
            if (!ok) {
                out.push_back(s);
                continue;
            }
            const std::string ind = indent_of(s.text), i1 = ind + "  ", i2 = ind + "    ";
            const std::string rows = u.in_ty.dims[0], chunks = std::to_string(std::stoll(u.in_ty.dims[1]) / 4);
            const std::string in_t = u.in_ty.str(), out_t = u.out_ty.str();
            const std::string e = fresh("init"), lb = fresh("c0"), st = fresh("c1"), ub0 = fresh("rows"), ub1 = fresh("chunks");
            out.push_back(mk(ind + e + " = tensor.empty() : " + out_t));
            out.push_back(mk(ind + lb + " = arith.constant 0 : index"));
            out.push_back(mk(ind + st + " = arith.constant 1 : index"));
            out.push_back(mk(ind + ub0 + " = arith.constant " + rows + " : index"));
            out.push_back(mk(ind + ub1 + " = arith.constant " + chunks + " : index"));
            std::string t = ind + s.result + " = scf.for %k = " + lb + " to " + ub0 + " step " + st + " iter_args(%acc_k = " + e +
                            ") -> (" + out_t + ") {\n";
            t += i1 + "%row = scf.for %ch = " + lb + " to " + ub1 + " step " + st + " iter_args(%acc = %acc_k) -> (" + out_t + ") {\n";
            t += i2 + "%four = arith.constant 4 : index\n";
            t += i2 + "%eight = arith.constant 8 : index\n";
            t += i2 + "%col = arith.muli %ch, %four : index\n";
            t += i2 + "%ocol = arith.muli %ch, %eight : index\n";
            for (int b = 1; b < 4; ++b) {
                t += i2 + "%off" + std::to_string(b) + " = arith.constant " + std::to_string(b) + " : index\n";
                t += i2 + "%col" + std::to_string(b) + " = arith.addi %col, %off" + std::to_string(b) + " : index\n";
            }
            t += i2 + "%b0 = tensor.extract " + u.in + "[%k, %col] : " + in_t + "\n";
            for (int b = 1; b < 4; ++b)
                t += i2 + "%b" + std::to_string(b) + " = tensor.extract " + u.in + "[%k, %col" + std::to_string(b) + "] : " + in_t + "\n";
            t += i2 + "%s8 = arith.constant 8 : i32\n";
            t += i2 + "%s16 = arith.constant 16 : i32\n";
            t += i2 + "%s24 = arith.constant 24 : i32\n";
            for (int b = 0; b < 4; ++b)
                t += i2 + "%e" + std::to_string(b) + " = arith.extui %b" + std::to_string(b) + " : i8 to i32\n";
            t += i2 + "%h1 = arith.shli %e1, %s8 : i32\n";
            t += i2 + "%w01 = arith.ori %e0, %h1 : i32\n";
            t += i2 + "%h2 = arith.shli %e2, %s16 : i32\n";
            t += i2 + "%w012 = arith.ori %w01, %h2 : i32\n";
            t += i2 + "%h3 = arith.shli %e3, %s24 : i32\n";
            t += i2 + "%w = arith.ori %w012, %h3 : i32\n";
            if (!use_prmt) {
                for (int n = 1; n < 8; ++n)
                    t += i2 + "%sh" + std::to_string(n) + " = arith.constant " + std::to_string(4 * n) + " : i32\n";
                t += i2 + "%mask = arith.constant 15 : i32\n";
                for (int n = 0; n < 8; ++n) {
                    const std::string ns = std::to_string(n);
                    std::string src = "%w";
                    if (n) {
                        t += i2 + "%r" + ns + " = arith.shrui %w, %sh" + ns + " : i32\n";
                        src = "%r" + ns;
                    }
                    t += i2 + "%m" + ns + " = arith.andi " + src + ", %mask : i32\n";
                    t += i2 + "%q" + ns + " = arith.trunci %m" + ns + " : i32 to i8\n";
                }
            } else {
                t += i2 + "%nib = arith.constant 252645135 : i32\n";  // 0x0F0F0F0F
                t += i2 + "%four32 = arith.constant 4 : i32\n";
                t += i2 + "%sel_lo = arith.constant 20800 : i32\n";   // 0x5140
                t += i2 + "%sel_hi = arith.constant 29538 : i32\n";   // 0x7362
                t += i2 + "%lo = arith.andi %w, %nib : i32\n";
                t += i2 + "%wsh = arith.shrui %w, %four32 : i32\n";
                t += i2 + "%hi = arith.andi %wsh, %nib : i32\n";
                t += i2 + "%c0123 = llvm.inline_asm \"prmt.b32 $0, $1, $2, $3;\", \"=r,r,r,r\" %lo, %hi, %sel_lo : (i32, i32, i32) -> i32\n";
                t += i2 + "%c4567 = llvm.inline_asm \"prmt.b32 $0, $1, $2, $3;\", \"=r,r,r,r\" %lo, %hi, %sel_hi : (i32, i32, i32) -> i32\n";
                for (int b = 1; b < 4; ++b)
                    t += i2 + "%bs" + std::to_string(b) + " = arith.constant " + std::to_string(8 * b) + " : i32\n";
                for (int n = 0; n < 8; ++n) {
                    const std::string ns = std::to_string(n), word = n < 4 ? "%c0123" : "%c4567";
                    std::string src = word;
                    if (n % 4) {
                        t += i2 + "%r" + ns + " = arith.shrui " + word + ", %bs" + std::to_string(n % 4) + " : i32\n";
                        src = "%r" + ns;
                    }
                    t += i2 + "%q" + ns + " = arith.trunci " + src + " : i32 to i8\n";
                }
            }
            std::string acc = "%acc";
            for (int n = 0; n < 8; ++n) {
                const std::string ns = std::to_string(n);
                std::string col = "%ocol";
                if (n) {
                    t += i2 + "%oo" + ns + " = arith.constant " + ns + " : index\n";
                    t += i2 + "%oc" + ns + " = arith.addi %ocol, %oo" + ns + " : index\n";
                    col = "%oc" + ns;
                }
                t += i2 + "%ins" + ns + " = tensor.insert %q" + ns + " into " + acc + "[%k, " + col + "] : " + out_t + "\n";
                acc = "%ins" + ns;
            }
            t += i2 + "scf.yield " + acc + " : " + out_t + "\n";
            t += i1 + "}\n";
            t += i1 + "scf.yield %row : " + out_t + "\n";
            t += ind + "}";
            out.push_back(mk(t));
        }
        f.body.swap(out);
    }
}

// --lower-dequant-to-arith (lib/Transforms/LowerDequantToArith.cpp:60-164): sitofp, sitofp, subf, mulf in f16
// with the rank-0 scale and zero point broadcast.
void pass_lower_dequant_to_arith(Module &mod) {
    for (auto &c : mod.chunks) {
        if (!c.is_func) continue;
        Func &f = c.func;
        std::vector<Stmt> out;
        for (const Stmt &s : f.body) {
            Dequant d;
            if (s.op == "qf.dequant") d = parse_dequant(s);
            if (!d.ok || d.out_ty.elem != "f16" || d.scale_ty != "tensor<f16>" || d.zp_ty != "tensor<i8>") {
                out.push_back(s);
                continue;
            }
            generic_dequant(indent_of(s.text), s.result, d.in, d, /*mask*/ false, /*zp*/ true, out);
        }
        f.body.swap(out);
    }
}

const std::set<std::string> kReferenceOnlyPasses = {
    "register-layout-aware-unpack", "quantforge-tiling",
    "quantforge-vectorization", "quantforge-gpu-mapping", "quantforge-bufferize", "quantforge-smem-promotion",
    "quantforge-swizzle-load", "quantforge-lower-to-nvvm"};

struct PassSpec {
    std::string name;
    int bitwidth = 8;
};

void add_pass(std::vector<PassSpec> &passes, const std::string &name, const std::string &opts) {
    PassSpec p;
    p.name = name;
    static const std::regex re(R"(qf-bitwidth\s*=\s*([0-9]+))");
    std::smatch m;
    if (std::regex_search(opts, m, re)) p.bitwidth = std::stoi(m[1]);
    passes.push_back(p);
}

void parse_pipeline(std::vector<PassSpec> &passes, const std::string &pipe) {
    // builtin.module(func.func(pass{opt=v},pass2)) : take the innermost list
    static const std::regex re(R"(([a-z][a-z0-9\-]*)(\{[^}]*\})?)");
    std::string inner = pipe;
    for (const char *wrap : {"builtin.module(", "func.func("}) {
        size_t p = inner.find(wrap);
        if (p != std::string::npos) {
            inner = inner.substr(p + std::string(wrap).size());
            size_t q = inner.rfind(')');
            if (q == std::string::npos) die("malformed -pass-pipeline");
            inner = inner.substr(0, q);
        }
    }
    for (auto it = std::sregex_iterator(inner.begin(), inner.end(), re); it != std::sregex_iterator(); ++it)
        add_pass(passes, (*it)[1], (*it)[2]);
}

}  // namespace

int main(int argc, char **argv) {
    std::vector<PassSpec> passes;
    std::string input = "-", output;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "-o" && i + 1 < argc) {
            output = argv[++i];
        } else if (a.rfind("-pass-pipeline=", 0) == 0 || a.rfind("--pass-pipeline=", 0) == 0) {
            std::string v = a.substr(a.find('=') + 1);
            if (!v.empty() && (v.front() == '\'' || v.front() == '"')) v = v.substr(1, v.size() - 2);
            parse_pipeline(passes, v);
        } else if (a == "--help" || a == "-h") {
            std::cout << "quantforge-opt (B200 runtime build): --convert-linalg-to-quantforge --fuse-unpack-dequant "
                         "--canonicalize-dequant-zp --lower-qf-to-runtime [-pass-pipeline=...] [-o out] [file|-]\n";
            return 0;
        } else if (a.rfind("--", 0) == 0) {
            std::string name = a.substr(2), opts;
            size_t eq = name.find('=');
            if (eq != std::string::npos) {
                opts = name.substr(0, eq) == "qf-bitwidth" ? name : "";
                if (!opts.empty()) {  // "--qf-bitwidth=4" applies to the last convert pass given
                    for (auto &p : passes)
                        if (p.name == "convert-linalg-to-quantforge") p.bitwidth = std::stoi(name.substr(eq + 1));
                    continue;
                }
                name = name.substr(0, eq);
            }
            add_pass(passes, name, opts);
        } else {
            input = a;
        }
    }
    Module mod;
    if (input == "-") {
        mod = parse(std::cin);
    } else {
        std::ifstream in(input);
        if (!in) die("cannot open " + input);
        mod = parse(in);
    }
    for (const auto &p : passes) {
        if (p.name == "convert-linalg-to-quantforge") {
            pass_convert(mod, p.bitwidth);
        } else if (p.name == "fuse-unpack-dequant") {
            pass_fuse(mod);
        } else if (p.name == "canonicalize-dequant-zp") {
            pass_canonicalize_zp(mod);
        } else if (p.name == "lower-qf-to-runtime") {
            pass_lower_to_runtime(mod);
        } else if (p.name == "lower-unpack-to-arith") {
            pass_lower_unpack_to_arith(mod);
        } else if (p.name == "lower-unpack-branch-free") {
            pass_branch_free(mod, false);
        } else if (p.name == "fuse-unpack-dequant-branch-free") {
            pass_branch_free(mod, true);
        } else if (p.name == "lower-unpack-to-nvvm") {
            pass_lower_unpack_loops(mod, false);
        } else if (p.name == "lower-unpack-to-prmt") {
            pass_lower_unpack_loops(mod, true);
        } else if (p.name == "lower-dequant-to-arith") {
            pass_lower_dequant_to_arith(mod);
        } else if (kReferenceOnlyPasses.count(p.name)) {
            die("pass '" + p.name + "' is not part of this build (generic GPU code generation scaffolding: tile shapes, "
                "staging, swizzle and launch geometry live inside the hand-written kernels)");
        } else {
            die("unknown pass '" + p.name + "'");
        }
    }
    if (output.empty()) {
        print(mod, std::cout);
    } else {
        std::ofstream os(output);
        if (!os) die("cannot write " + output);
        print(mod, os);
    }
    return 0;
}
