"""Expands the reference's kernel templates without Ruby (TEST INFRASTRUCTURE, not product).

The reference generates `ext/cumo/narray/types/<type>_kernel.cu` with a Ruby program
(`ext/cumo/narray/gen/cogen_kernel.rb`): it evaluates `gen/def/<type>.rb` and `gen/spec.rb`
into a list of method definitions (`gen/narray_def.rb`, `gen/erbpp2.rb`), and renders for each
of them the ERB template `gen/tmpl/<erb_base>_kernel.cu` if there is one, all into one
translation unit (`gen/tmpl/lib_kernel.cu`).  There is no Ruby where this project is built, so
this module restates that generator in Python, narrowly: the handful of Ruby constructs that
`spec.rb`, the `def/*.rb` files and the kernel templates actually use.  Anything else fails
loudly instead of being guessed.

It reads the reference where it lies (a checkout passed as `ref_root`), and is used by
  * oracle/build_ref_kernels.py -- compiles the expanded kernels into oracle/_ref/ as the
    "reference's own kernels on the same GPU" baseline and second oracle;
  * tests/golden/make_abi_manifest.py -- writes the list of launch functions (name and
    argument types) that the reference's generated kernel units define.
Nothing the library ships imports it.
"""
from __future__ import annotations

import re
from pathlib import Path

TYPES = ("sfloat", "dfloat", "int32", "int64")


# --------------------------------------------------------------------------------------
# Ruby expression subset -> Python
# --------------------------------------------------------------------------------------
def _interp_string(body: str) -> str:
    """A Ruby double-quoted string body with #{...} interpolation as a Python expression."""
    parts, pos = [], 0
    for m in re.finditer(r"#\{([^}]*)\}", body):
        if m.start() > pos:
            parts.append(repr(body[pos:m.start()]))
        parts.append(f"str({rb_expr(m.group(1))})")
        pos = m.end()
    if pos < len(body):
        parts.append(repr(body[pos:]))
    return "(" + " + ".join(parts or ["''"]) + ")"


def rb_expr(src: str) -> str:
    """Translate one Ruby expression of the kind the templates use."""
    s = src.strip()
    strings: list[str] = []

    def stash(py: str) -> str:
        strings.append(py)
        return f"\x00{len(strings) - 1}\x00"

    s = re.sub(r'"((?:[^"\\]|\\.)*)"', lambda m: stash(_interp_string(m.group(1))), s)
    s = re.sub(r"'((?:[^'\\]|\\.)*)'", lambda m: stash(repr(m.group(1))), s)
    s = re.sub(r"%w\[([^\]]*)\]", lambda m: stash("[" + ",".join(repr(w) for w in m.group(1).split()) + "]"), s)
    s = re.sub(r"defined\?\(\$(\w+)\)", lambda m: f"({m.group(1)!r} in G)", s)
    s = re.sub(r"\$(\w+)", lambda m: f"G[{m.group(1)!r}]", s)
    s = re.sub(r"load_erb\((\x00\d+\x00)\)\.result\(binding\)", r"load_erb(\1)", s)
    s = re.sub(r"\((\w+)\.\.(\w+)\)", r"list(range(\1, \2 + 1))", s)
    s = s.replace(".to_a", "")
    s = re.sub(r"\bc_func\([^)]*\)", "c_func", s)                  # the argument only sets the arity of the Ruby binding
    s = re.sub(r"\.result\b(?!\()", ".result()", s)
    s = re.sub(r"<<\s*(\x00\d+\x00)", r"+ [\1]", s)
    # X.include?(Y) / X.include? Y
    s = re.sub(r"((?:\x00\d+\x00)|[\w.]+)\.include\?\s*\(?\s*((?:\x00\d+\x00)|\w+)\s*\)?", r"(\2 in \1)", s)
    # (c ? a : b)
    s = re.sub(r"\(([^?()]+)\?\s*([^:]+):\s*([^)]+)\)", r"((\2) if (\1) else (\3))", s)
    s = re.sub(r"(?<![\w)])!\s*(?=[\w(])", "not ", s)
    s = s.replace("&&", " and ").replace("||", " or ")
    s = re.sub(r"(?<![\w:]):(\w+)", r"'\1'", s)                      # :symbol
    s = re.sub(r"\bnil\b", "None", s)
    s = re.sub(r"\btrue\b", "True", s)
    s = re.sub(r"\bfalse\b", "False", s)
    s = re.sub(r"\x00(\d+)\x00", lambda m: strings[int(m.group(1))], s)
    return s


# --------------------------------------------------------------------------------------
# ERB subset
# --------------------------------------------------------------------------------------
class _Scope(dict):
    """Name lookup of a template: its own loop variables, then the method object and its parents."""

    def __init__(self, node, helpers):
        super().__init__(helpers)
        self.node = node

    def __missing__(self, key):
        v = self.node.get(key)
        if v is _MISSING:
            raise KeyError(key)                      # the lookup goes on to the builtins, then fails as a NameError
        return v


_MISSING = object()


def erb_to_python(text: str) -> str:
    """An ERB template (`<% code %>`, `<%= value %>`) as the body of a Python function that appends to `out`."""
    lines, depth = [], 0

    def emit(code):
        lines.append("    " * depth + code)

    pos = 0
    for m in re.finditer(r"<%(=?)(.*?)%>", text, re.S):
        if m.start() > pos:
            emit(f"out.append({text[pos:m.start()]!r})")
        pos = m.end()
        body = m.group(2).strip()
        if m.group(1) == "=":
            emit(f"out.append(_s({rb_expr(body)}))")
            continue
        if body.startswith("#") or not body:
            continue
        mm = re.fullmatch(r"(.*)\.each\s+do\s*\|([^|]*)\|", body, re.S)
        if mm:
            emit(f"for {mm.group(2).strip()} in {rb_expr(mm.group(1))}:")
            depth += 1
            emit("pass")
        elif body.startswith("if "):
            emit(f"if {rb_expr(body[3:])}:")
            depth += 1
            emit("pass")
        elif body.startswith("unless "):
            emit(f"if not ({rb_expr(body[7:])}):")
            depth += 1
            emit("pass")
        elif body.startswith("elsif "):
            depth -= 1
            emit(f"elif {rb_expr(body[6:])}:")
            depth += 1
            emit("pass")
        elif body == "else":
            depth -= 1
            emit("else:")
            depth += 1
            emit("pass")
        elif body == "end":
            depth -= 1
            if depth < 0:
                raise SyntaxError("unbalanced `end` in template")
        else:
            mm = re.fullmatch(r"(\$?\w+)\s*=\s*(.*)", body, re.S)
            if not mm:
                raise SyntaxError(f"unsupported Ruby in template: {body!r}")
            target = f"G[{mm.group(1)[1:]!r}]" if mm.group(1).startswith("$") else mm.group(1)
            emit(f"{target} = {rb_expr(mm.group(2))}")
    if pos < len(text):
        emit(f"out.append({text[pos:]!r})")
    if depth != 0:
        raise SyntaxError("unterminated block in template")
    return "\n".join(lines)


# --------------------------------------------------------------------------------------
# The generator's object tree (gen/erbpp2.rb, gen/narray_def.rb), restated
# --------------------------------------------------------------------------------------
class Node:
    def __init__(self, gen, parent, erb_base, **opts):
        self.gen, self.parent, self.opts, self.children = gen, parent, dict(opts), []
        if erb_base:
            self.opts["erb_base"] = erb_base
        if parent is not None:
            parent.children.append(self)

    def describe(self):
        return f"{self.opts.get('erb_base')}:{self.opts.get('name')}"

    # erbpp2.rb:27-38: a method of the object, then its options, then the parent's
    def get(self, key):
        fn = getattr(self, "rb_" + key, None)
        if fn is not None:
            return fn()
        if key in self.opts:
            return self.opts[key]
        if self.parent is not None:
            return self.parent.get(key)
        return _MISSING

    def result(self):
        base = self.opts.get("erb_base")
        return self.gen.render(base, self) if base else ""


class MethodNode(Node):
    # erbpp2.rb:232-256
    def rb_c_name(self):
        return self.opts["name"].replace("?", "_p").replace("!", "_bang").replace("=", "_set")

    def rb_c_func(self):
        s = "_s" if self.opts.get("singleton") else ""
        return f"{self.parent.get('name')}{s}_{self.rb_c_name()}"

    def rb_c_iter(self):
        return "iter_" + self.rb_c_func()


class StoreNode(MethodNode):
    # narray_def.rb:228-231: named after the class two levels up
    def rb_c_func(self):
        return f"{self.parent.parent.get('name')}_store_{self.opts['name']}"


class ContainerNode(MethodNode):
    def rb_method_code(self):                       # erbpp2.rb:197-199
        return "\n".join(c.result() for c in self.children)


class ClassNode(ContainerNode):
    def rb_type_name(self):                         # narray_def.rb:117-119
        return self.opts.get("type_name") or self.opts["class_name"].lower()


# narray_def.rb:7-91: DSL word -> (template, option names of the positional arguments after the method name)
_DSL = {
    "binary": ("binary", ["op"]), "binary2": ("binary2", ["op"]), "unary": ("unary", ["op"]),
    "unary2": ("unary2", ["dtype", "result_class"]), "set2": ("set2", ["dtype", "result_class"]),
    "cond_binary": ("cond_binary", ["op"]), "cond_unary": ("cond_unary", []),
    "bit_count": ("bit_count", []), "bit_count_cpu": ("bit_count_cpu", []), "bit_reduce": ("bit_reduce", ["init_bit"]),
    "accum": ("accum", ["dtype", "result_class"]), "accum_index": ("accum_index", []), "accum_arg": ("accum_arg", []),
    "cum": ("cum", ["cmacro"]), "accum_binary": ("accum_binary", ["op"]),
}


class Generator:
    """One element type's generator run: def/<type>.rb + spec.rb evaluated into a tree, templates rendered from it."""

    def __init__(self, ref_root, type_name: str, suffix: str = "_kernel.cu"):
        self.gen_dir = Path(ref_root) / "ext/cumo/narray/gen"
        self.suffix = suffix
        self.type_name = type_name
        self.G: dict = {}                            # Ruby's $globals, shared by all templates of the run
        self.erb_dirs = [self.gen_dir / "tmpl"]
        if type_name == "bit":                       # cogen_kernel.rb:34-36
            self.erb_dirs.insert(0, self.gen_dir / "tmpl_bit")
        indexer_h = (Path(ref_root) / "ext/cumo/include/cumo/indexer.h").read_text()
        ndim = int(re.search(r"CUMO_NA_INDEXER_OPTIMIZED_NDIM (\d+)", indexer_h).group(1))
        self.lib = Node(self, None, "lib", type_name=type_name, lib_name="cumo_" + type_name, opt_indexer_ndim=ndim)
        self.klass = ClassNode(self, self.lib, "class")
        self._eval_def(self.gen_dir / "def" / f"{type_name}.rb")
        self._eval_spec(self.gen_dir / "spec.rb")
        self._compiled: dict[str, object] = {}

    # ---- def/<type>.rb: `set key: value` lines; the upcast tables are not needed here ----
    def _eval_def(self, path):
        for line in path.read_text().splitlines():
            m = re.match(r"\s*set\s+(\w+):\s*(.+?)\s*$", line)
            if m:
                self.klass.opts[m.group(1)] = eval(rb_expr(m.group(2)))

    # ---- spec.rb ----
    def _flag(self, expr, extra):
        scope = _Scope(self.klass, extra)
        return bool(eval(rb_expr(expr), {}, scope))

    def _eval_spec(self, path):
        # frames: [executing?, ever_taken?, kind, saved_target]
        frames, target, local = [], self.klass, {}
        for raw in path.read_text().splitlines():
            line = re.sub(r"\s+#.*$", "", raw).strip()
            if not line or line.startswith("#"):
                continue
            live = all(f[0] for f in frames)
            if re.match(r"if\b", line):
                ok = live and self._flag(line[2:], local)
                frames.append([ok, ok, "if", None])
                continue
            if line == "else":
                f = frames[-1]
                f[0] = (not f[1]) and all(g[0] for g in frames[:-1])
                continue
            if re.match(r"end\b", line):
                f = frames.pop()
                if f[2] == "block" and f[3] is not None:
                    target = f[3]
                continue
            m = re.match(r"(.*\S)\s+do$", line)
            if m:
                saved = None
                if live:
                    saved, head = target, m.group(1)
                    if head.startswith("def_module"):
                        target = ContainerNode(self, self.lib, "module", singleton=False)
                    else:
                        target = self._statement(head, target, local, container=True)
                frames.append([live, live, "block", saved])
                continue
            if not live:
                continue
            m = re.match(r"(.*\S)\s+if\s+(.*)$", line)
            if m and not line.startswith("def_const"):
                if not self._flag(m.group(2), local):
                    continue
                line = m.group(1)
            m = re.match(r"(\w+)\s*=\s*(.*)$", line)
            if m:                                    # fn = get(:full_class_name), is_c = is_complex ...
                rhs = re.sub(r"get\(:(\w+)\)", r"\1", m.group(2))
                local[m.group(1)] = eval(rb_expr(rhs), {}, _Scope(self.klass, local))
                continue
            self._statement(line, target, local)
        if frames:
            raise SyntaxError("spec.rb: unterminated block")

    def _args(self, text, local):
        """Positional arguments and key: value options of a DSL call."""
        pos, opts = [], {}
        for part in re.findall(r'(?:[^,"\']|"[^"]*"|\'[^\']*\')+', text):
            part = part.strip()
            if not part:
                continue
            m = re.match(r"(\w+):\s*(.*)$", part)
            if m:
                opts[m.group(1)] = eval(rb_expr(m.group(2)), {}, _Scope(self.klass, local))
            else:
                pos.append(eval(rb_expr(part), {}, _Scope(self.klass, local)))
        return pos, opts

    def _statement(self, line, target, local, container=False):
        m = re.match(r"(\w+)\s*(.*)$", line)
        word, rest = m.group(1), m.group(2)
        if word in ("def_id", "def_const", "def_alias", "undef_method", "undef_singleton_method", "extend", "def_alloc_func"):
            return None
        pos, opts = self._args(rest, local)
        cls = ContainerNode if container else MethodNode
        if word == "set":
            target.opts.update(opts)
        elif word in _DSL:
            tmpl, names = _DSL[word]
            if word in ("binary", "binary2", "accum_binary", "cond_binary") and len(pos) == 1:
                pos.append(pos[0])                   # the operator defaults to the method name
            return cls(self, target, tmpl, name=pos[0], **dict(zip(names, pos[1:])), **opts)
        elif word == "pow":
            return cls(self, target, "pow", name="pow", op="**")
        elif word in ("def_method", "def_singleton_method"):
            return cls(self, target, pos[1] if len(pos) > 1 else pos[0], name=pos[0], singleton=word == "def_singleton_method", **opts)
        elif word == "def_module_function":
            return cls(self, target, pos[1] if len(pos) > 1 else pos[0], name=pos[0], singleton=True, **opts)
        elif word == "math":                         # narray_def.rb:95-111
            n = pos[1] if len(pos) > 1 else 1
            tmpl = pos[2] if len(pos) > 2 else {1: "unary_s", 2: "binary_s", 3: "ternary_s"}[n]
            return cls(self, target, tmpl, name=pos[0], singleton=True, **opts)
        elif word == "store_from":                   # narray_def.rb:196-205
            cname = pos[0]
            return StoreNode(self, target, "store_bit" if cname == "Bit" else "store_from", name=cname.lower(), type_name=cname,
                             type_var="cumo_c" + cname, dtype=pos[1] if len(pos) > 1 else None, macro=pos[2] if len(pos) > 2 else None)
        elif word == "store_numeric":
            return StoreNode(self, target, "store_numeric", name="numeric")
        elif word == "store_array":
            return StoreNode(self, target, "store_array", name="array")
        elif word == "qsort":
            return cls(self, target, "qsort", name="qsort", type_name=pos[0], dtype=pos[1], dcast=pos[2], suffix=pos[3] if len(pos) > 3 else "")
        else:
            raise SyntaxError(f"spec.rb: unknown statement {line!r}")
        return None

    # ---- rendering ----
    def template_path(self, base):
        for d in self.erb_dirs:
            p = d / (base + self.suffix)
            if p.exists():
                return p
        return None

    def render(self, base, node) -> str:
        path = self.template_path(base)
        if path is None:
            return ""                                # erbpp2.rb:86-92: no template of that name for this suffix
        if base not in self._compiled:
            body = ["if True:"] + ["    " + l for l in erb_to_python(path.read_text()).splitlines()] + ["    pass"]
            self._compiled[base] = compile("\n".join(body), str(path), "exec")
        out: list[str] = []
        helpers = {"out": out, "_s": lambda v: "" if v is None else str(v), "G": self.G,
                   "load_erb": lambda b: self.render(b, node), "children": node.children}
        # template variables are free names of the translated code: they resolve through the scope mapping
        exec(self._compiled[base], {"__builtins__": __builtins__}, _Scope(node, helpers))
        return "".join(out)

    def methods(self):
        """Every method node of the run, in definition order (class methods, store sources, math functions)."""
        def walk(n):
            for c in n.children:
                yield c
                yield from walk(c)
        return list(walk(self.lib))

    def kernel_unit(self, only: set[str] | None = None) -> str:
        """The text of types/<type>_kernel.cu, optionally keeping only the templates in `only` (by erb_base)."""
        if only is None:
            return self.lib.result()
        head = '#include "cumo/narray_kernel.h"\n#include "cumo/indexer.h"\n#include "cumo/reduce_kernel.h"\n' \
               f'#include <cumo/types/{self.type_name}_kernel.h>\n\nextern "C" {{\n'
        parts = []
        for top in self.lib.children:                # the class, then the math module
            for c in top.children:
                if c.opts.get("erb_base") in only or (c.opts.get("erb_base") == "store" and "store_from" in only):
                    if c.opts.get("erb_base") == "store":
                        parts.extend(g.result() for g in c.children if g.opts.get("erb_base") in only)
                    else:
                        parts.append(c.result())
        return head + "\n\n".join(parts) + "\n}\n"


# --------------------------------------------------------------------------------------
# Launch functions defined by a kernel unit
# --------------------------------------------------------------------------------------
_C_TYPE = {"sfloat": "float", "dfloat": "double", "int32": "int32_t", "int64": "int64_t", "bit": "CUMO_BIT_DIGIT"}


def launch_functions(unit_text: str, type_name: str):
    """(name, return type, [argument types]) of every non-static function a kernel unit defines at file scope whose
    name ends in `_kernel_launch` (or is `cumo_bit_where_scratch_new`); `dtype` is spelt as the C type."""
    text = re.sub(r"/\*.*?\*/", "", unit_text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = []
    for m in re.finditer(r"^(?!static)([A-Za-z_][\w ]*?[\w*])\s*\n?\s*\b(cumo_\w+)\s*\(([^)]*)\)\s*\{", text, re.M):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)
        if "__global__" in ret or ret.startswith("static") or not (name.endswith("_kernel_launch") or name == "cumo_bit_where_scratch_new"):
            continue
        types = []
        for a in args.split(","):
            a = a.strip()
            if not a or a == "void":
                continue
            a = re.sub(r"\s*\b\w+$", "", a) if re.search(r"[\w*]\s+\**\w+$|\*\w+$", a) else a    # drop the parameter name
            a = re.sub(r"\s*\*\s*", "*", a).strip()
            a = re.sub(r"\bdtype\b", _C_TYPE[type_name], a)
            types.append(a)
        out.append((name, re.sub(r"\s*\*\s*", "*", ret), types))
    return out
