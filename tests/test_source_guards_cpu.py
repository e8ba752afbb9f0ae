"""Source guards: properties of the sources themselves that no run on a CPU box can show, checked by reading them
(the idea of the reference's dev/validate_*_source.py scripts, e.g. dev/validate_nccl_source.py:1-349, applied to this
framework's own rules)."""
import os
import re

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(REPO, "llm_kittens_b200")
CSRC = os.path.join(PKG, "csrc")


def _read(path):
    with open(path, encoding="utf-8") as f:
        return f.read()


def _files(root, exts):
    for d, _, names in os.walk(root):
        if "_lib" in d or "__pycache__" in d:
            continue
        for n in sorted(names):
            if n.endswith(exts):
                yield os.path.join(d, n)


def _strip_comments(src):
    src = re.sub(r"/\*.*?\*/", " ", src, flags=re.S)
    return re.sub(r"//[^\n]*", " ", src)


def test_every_entry_point_called_from_python_is_exported_by_the_cuda_sources():
    exported = set()
    for path in _files(CSRC, (".cu", ".cpp", ".cuh", ".h")):
        exported |= set(re.findall(r"\b(llmk_[a-z0-9_]+)\s*\(", _read(path)))
    called = {}
    for path in list(_files(PKG, (".py",))) + [os.path.join(REPO, "bench.py"), os.path.join(REPO, "__graft_entry__.py")]:
        src = _read(path)
        for name in re.findall(r"""(?:N|_native|native)\.call\(\s*["'](llmk_[a-z0-9_]+)["']""", src):
            called.setdefault(name, path)
        for name in re.findall(r"""lib\(\)\.(llmk_[a-z0-9_]+)\b""", src):
            called.setdefault(name, path)
    assert len(called) > 60, "the scan found suspiciously few call sites"
    missing = {n: p for n, p in called.items() if n not in exported}
    assert not missing, f"called from Python but defined nowhere in csrc: {missing}"


def test_no_copy_into_shared_memory_is_broadcast_to_the_ctas_of_a_cluster():
    """The only use of the cluster-broadcast qualifier in the kernels is the tcgen05.commit arrival (an mbarrier signal,
    no data). The qualifier is spelled in two halves here so that this file does not contain it."""
    qualifier = "multi" + "cast::" + "cluster"
    for path in _files(CSRC, (".cu", ".cuh")):
        code = _strip_comments(_read(path))
        for m in re.finditer(re.escape(qualifier), code):
            line = code[code.rfind("\n", 0, m.start()) + 1: code.find("\n", m.end())]
            assert "tcgen05.commit" in line, f"{path}: {line.strip()}"


def test_device_code_has_no_trap_and_every_polling_loop_has_a_time_limit():
    for path in _files(CSRC, (".cu", ".cuh")):
        code = _strip_comments(_read(path))
        assert "__trap" not in code and "asm(\"trap" not in code and not re.search(r"(?<![\w])assert\(", code), path
        # every loop that polls memory written by another kernel, CTA or GPU sits next to a timer read and an abort path
        for m in re.finditer(r"while\s*\([^)]*(ld_acquire|ld_shared_acquire|ld_volatile|mbar_test|mbar_poll)", code):
            window = code[m.start(): m.start() + 1500]
            assert re.search(r"globaltimer_ns|now_ns\(\)|clock64", window), f"{path}: polling loop without a time limit near: {window[:80]!r}"
        for m in re.finditer(r"while\s*\(\s*true\s*\)", code):
            window = code[m.start(): m.start() + 1200]
            assert re.search(r"globaltimer_ns|now_ns\(\)|clock64|break|return", window), f"{path}: endless loop near {window[:80]!r}"


def test_every_profiler_command_line_leaves_the_clocks_alone():
    hits = 0
    for path in list(_files(PKG, (".py",))) + list(_files(os.path.join(REPO, "profiles"), (".md",))) + [os.path.join(REPO, "README.md")]:
        src = _read(path)
        for m in re.finditer(r"""(?<![\w`.])ncu(?:["',\s]+)--""", src):
            window = src[m.start(): m.start() + 700]
            assert "--clock-control" in window and "none" in window, f"{path}: ncu without --clock-control none near {window[:80]!r}"
            hits += 1
    assert hits >= 5


def test_build_targets_sm_100a_only_and_keeps_line_info():
    src = _read(os.path.join(PKG, "build.py"))
    assert "arch=compute_100a,code=sm_100a" in src and "-lineinfo" in src
    assert not re.search(r"sm_(80|86|89|90a?|120)\b", src)


def test_nothing_committed_depends_on_the_scratch_folder():
    for path in list(_files(PKG, (".py",))) + list(_files(os.path.join(REPO, "tests"), (".py",))) + [os.path.join(REPO, "bench.py")]:
        if path.endswith("test_source_guards_cpu.py"):
            continue
        assert "_work/" not in _read(path) and "_work\\" not in _read(path), path


def test_no_function_refers_to_a_name_that_does_not_exist():
    """Most of the package only runs on a GPU; a misspelt or forgotten name in such a function would not show in the
    CPU tier. The symbol tables say which names every function takes from the module's globals: each must exist there
    (after import) or be a builtin."""
    import builtins
    import importlib
    import importlib.util
    import pkgutil
    import symtable

    import llm_kittens_b200

    def walk(table, module_names, path, problems):
        for child in table.get_children():
            if child.get_type() == "function":
                for sym in child.get_symbols():
                    if sym.is_global() and sym.is_referenced() and not sym.is_assigned():
                        name = sym.get_name()
                        if name not in module_names and not hasattr(builtins, name):
                            problems.append(f"{path}: {child.get_name()}() uses undefined name {name!r}")
            walk(child, module_names, path, problems)

    problems = []
    mods = [m.name for m in pkgutil.walk_packages(llm_kittens_b200.__path__, "llm_kittens_b200.")]
    assert len(mods) > 40
    for name in mods:
        mod = importlib.import_module(name)
        path = mod.__file__
        walk(symtable.symtable(_read(path), path, "exec"), set(vars(mod)), os.path.relpath(path, REPO), problems)
    for path in (os.path.join(REPO, "bench.py"), os.path.join(REPO, "__graft_entry__.py")):
        spec = importlib.util.spec_from_file_location("_guard_" + os.path.basename(path)[:-3], path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        walk(symtable.symtable(_read(path), path, "exec"), set(vars(mod)), os.path.relpath(path, REPO), problems)
    assert not problems, "\n".join(problems)


def test_every_attribute_taken_from_a_module_of_the_package_exists():
    """``gemm.gemm_tn``, ``N.status_word``, ``moe_ops.combine_pull`` ...: where a name is bound by an import to a module
    (of this package or of the standard library) and an attribute is read from it, the attribute must exist. Catches a
    misspelt or renamed function in code that only runs on a GPU."""
    import ast
    import importlib
    import pkgutil
    import types

    import llm_kittens_b200

    problems = []
    files = []
    for info in pkgutil.walk_packages(llm_kittens_b200.__path__, "llm_kittens_b200."):
        files.append((importlib.import_module(info.name).__file__, info.name if info.ispkg else info.name.rsplit(".", 1)[0]))
    # the GPU tests and the benchmark use the package too, and do not run here either
    files += [(p, None) for p in _files(os.path.join(REPO, "tests"), (".py",))] + [(os.path.join(REPO, "bench.py"), None)]
    for file_path, package in files:
        tree = ast.parse(_read(file_path))
        bound = {}        # local name -> module object, from every import statement in the file (any scope)
        for node in ast.walk(tree):
            if isinstance(node, ast.ImportFrom):
                base = "." * node.level + (node.module or "")
                for al in node.names:
                    for target in (f"{base}.{al.name}" if node.module else f"{base}{al.name}",):
                        try:
                            m = importlib.import_module(target, package) if node.level else importlib.import_module(f"{node.module}.{al.name}")
                        except Exception:
                            continue
                        if isinstance(m, types.ModuleType):
                            bound[al.asname or al.name] = m
            elif isinstance(node, ast.Import):
                for al in node.names:
                    if "." not in al.name or al.asname:
                        try:
                            bound[al.asname or al.name] = importlib.import_module(al.name)
                        except Exception:
                            pass
        rebound = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store)}
        rebound |= {a.arg for n in ast.walk(tree) if isinstance(n, ast.arguments) for a in n.args + n.kwonlyargs}
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and isinstance(node.ctx, ast.Load):
                name = node.value.id
                if name in bound and name not in rebound and not hasattr(bound[name], node.attr):
                    owner = bound[name].__name__
                    if owner.startswith("llm_kittens_b200") or owner in ("os", "sys", "math", "ctypes", "json", "time", "struct"):
                        problems.append(f"{os.path.relpath(file_path, REPO)}:{node.lineno}: {name}.{node.attr} does not exist in {owner}")
    assert not problems, "\n".join(problems)


def test_calls_of_package_functions_fit_their_signatures():
    """``module.function(a, b, key=c)`` where the module is one of this package: the positional count and the keyword
    names must bind to the function's signature (calls with ``*args`` / ``**kwargs`` are skipped). A wrong keyword in
    code that only runs on a GPU would otherwise wait for a GPU to be found."""
    import ast
    import importlib
    import inspect
    import pkgutil
    import types

    import llm_kittens_b200

    files = []
    for info in pkgutil.walk_packages(llm_kittens_b200.__path__, "llm_kittens_b200."):
        files.append((importlib.import_module(info.name).__file__, info.name if info.ispkg else info.name.rsplit(".", 1)[0]))
    files += [(p, None) for p in _files(os.path.join(REPO, "tests"), (".py",))] + [(os.path.join(REPO, "bench.py"), None)]
    problems, checked = [], 0
    for file_path, package in files:
        tree = ast.parse(_read(file_path))
        bound = {}
        for node in ast.walk(tree):
            if isinstance(node, ast.ImportFrom):
                base = "." * node.level + (node.module or "")
                for al in node.names:
                    target = f"{base}.{al.name}" if node.module else f"{base}{al.name}"
                    try:
                        m = importlib.import_module(target, package) if node.level else importlib.import_module(f"{node.module}.{al.name}")
                    except Exception:
                        continue
                    if isinstance(m, types.ModuleType) and m.__name__.startswith("llm_kittens_b200"):
                        bound[al.asname or al.name] = m
        rebound = {n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store)}
        rebound |= {a.arg for n in ast.walk(tree) if isinstance(n, ast.arguments) for a in n.args + n.kwonlyargs}
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and isinstance(node.func.value, ast.Name)):
                continue
            name = node.func.value.id
            if name not in bound or name in rebound:
                continue
            fn = getattr(bound[name], node.func.attr, None)
            if not inspect.isfunction(fn):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords):
                continue
            try:
                inspect.signature(fn).bind(*[None] * len(node.args), **{k.arg: None for k in node.keywords})
                checked += 1
            except TypeError as e:
                problems.append(f"{os.path.relpath(file_path, REPO)}:{node.lineno}: {name}.{node.func.attr}(...): {e}")
    assert checked > 300, checked
    assert not problems, "\n".join(problems)


def test_native_calls_pass_as_many_arguments_as_the_c_entry_points_take():
    """``N.call("llmk_x", a, b, ...)`` appends the stream and calls through ctypes without prototypes: a missing or extra
    argument would not raise, it would shift every later parameter. The C signatures are read from the sources and
    compared with every call site."""
    import ast

    sigs = {}
    for path in _files(CSRC, (".cu", ".cpp")):
        code = _strip_comments(_read(path))
        for m in re.finditer(r"LLMK_API\s+[\w\s\*]+?\b(llmk_[a-z0-9_]+)\s*\(([^)]*)\)\s*\{", code):
            params = [p for p in m.group(2).split(",") if p.strip() and p.strip() != "void"]
            sigs[m.group(1)] = len(params)
    assert len(sigs) > 80, len(sigs)
    problems, checked = [], 0
    files = list(_files(PKG, (".py",))) + list(_files(os.path.join(REPO, "tests"), (".py",))) + [os.path.join(REPO, "bench.py")]
    for path in files:
        for node in ast.walk(ast.parse(_read(path))):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr == "call" and node.args):
                continue
            first = node.args[0]
            if not (isinstance(first, ast.Constant) and isinstance(first.value, str) and first.value.startswith("llmk_")):
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or node.keywords:
                continue
            name = first.value
            assert name in sigs, f"{path}:{node.lineno}: {name} has no definition with a body in csrc"
            passed = len(node.args) - 1 + 1          # the arguments after the name, plus the stream that call() appends
            checked += 1
            if passed != sigs[name]:
                problems.append(f"{os.path.relpath(path, REPO)}:{node.lineno}: {name} takes {sigs[name]} parameters, the call passes {passed}")
            # direct calls through the library handle (size queries and the like) pass exactly what they list
    direct = 0
    for path in files:
        for node in ast.walk(ast.parse(_read(path))):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr.startswith("llmk_") \
                    and node.func.attr in sigs and not node.keywords and not any(isinstance(a, ast.Starred) for a in node.args):
                direct += 1
                if len(node.args) != sigs[node.func.attr]:
                    problems.append(f"{os.path.relpath(path, REPO)}:{node.lineno}: {node.func.attr} takes {sigs[node.func.attr]} "
                                    f"parameters, the call passes {len(node.args)}")
    assert checked > 80 and direct > 10, (checked, direct)
    assert not problems, "\n".join(problems)


def test_calls_of_imported_functions_and_classes_fit_their_signatures():
    """The same for names imported directly (``from ..runtime.trainer import Trainer`` ... ``Trainer(model, zero_stage=1)``,
    ``generate(model, prompt, n, rng_state=s)``): constructor and function calls must bind."""
    import ast
    import importlib
    import inspect
    import pkgutil

    import llm_kittens_b200

    files = []
    for info in pkgutil.walk_packages(llm_kittens_b200.__path__, "llm_kittens_b200."):
        files.append((importlib.import_module(info.name).__file__, info.name if info.ispkg else info.name.rsplit(".", 1)[0]))
    files += [(p, None) for p in _files(os.path.join(REPO, "tests"), (".py",))] + [(os.path.join(REPO, "bench.py"), None)]
    problems, checked = [], 0
    for file_path, package in files:
        tree = ast.parse(_read(file_path))
        bound = {}
        for node in ast.walk(tree):
            if isinstance(node, ast.ImportFrom) and (node.level or (node.module or "").startswith("llm_kittens_b200")):
                try:
                    m = importlib.import_module("." * node.level + (node.module or ""), package) if node.level else importlib.import_module(node.module)
                except Exception:
                    continue
                for al in node.names:
                    obj = getattr(m, al.name, None)
                    if inspect.isfunction(obj) or inspect.isclass(obj):
                        bound[al.asname or al.name] = obj
        stores = [n.id for n in ast.walk(tree) if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store)]
        stores += [n.name for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.ClassDef))]
        for node in ast.walk(tree):
            if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in bound) or node.func.id in stores:
                continue
            if any(isinstance(a, ast.Starred) for a in node.args) or any(k.arg is None for k in node.keywords):
                continue
            obj = bound[node.func.id]
            try:
                sig = inspect.signature(obj)
            except (TypeError, ValueError):
                continue
            try:
                sig.bind(*[None] * len(node.args), **{k.arg: None for k in node.keywords})
                checked += 1
            except TypeError as e:
                problems.append(f"{os.path.relpath(file_path, REPO)}:{node.lineno}: {node.func.id}(...): {e}")
    assert checked > 150, checked
    assert not problems, "\n".join(problems)
