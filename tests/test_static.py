"""Static checks of the Python files that only run on GPU boxes (bench.py, benchmarks/, the GPU paths of the
package): every file compiles, and no name is read that the file never binds (a typo there would otherwise
show only on a GPU).  Plus the reference arm of the benchmark, which must answer without a GPU."""

import ast
import builtins
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _python_files():
    for top in ("bench.py", "__graft_entry__.py", "benchmarks", "examples", "moodist_b200", "tests"):
        path = os.path.join(ROOT, top)
        if os.path.isfile(path):
            yield path
        for d, _, files in os.walk(path):
            for f in files:
                if f.endswith(".py"):
                    yield os.path.join(d, f)


def _bound_names(tree):
    bound = set(dir(builtins)) | {"__file__", "__name__", "__doc__", "__class__"}
    for node in ast.walk(tree):
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
            bound.add(node.name)
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.Lambda)):
            a = node.args
            for arg in a.posonlyargs + a.args + a.kwonlyargs + ([a.vararg] if a.vararg else []) + ([a.kwarg] if a.kwarg else []):
                bound.add(arg.arg)
        elif isinstance(node, ast.Name) and isinstance(node.ctx, (ast.Store, ast.Del)):
            bound.add(node.id)
        elif isinstance(node, (ast.Import, ast.ImportFrom)):
            for alias in node.names:
                bound.add((alias.asname or alias.name).split(".")[0])
        elif isinstance(node, ast.ExceptHandler) and node.name:
            bound.add(node.name)
        elif isinstance(node, (ast.Global, ast.Nonlocal)):
            bound.update(node.names)
        elif isinstance(node, ast.MatchAs) and node.name:
            bound.add(node.name)
    return bound


def test_every_python_file_compiles_and_reads_only_names_it_binds():
    problems = []
    for path in sorted(set(_python_files())):
        src = open(path).read()
        try:
            tree = ast.parse(src, filename=path)
            compile(src, path, "exec")
        except SyntaxError as e:
            problems.append(f"{path}: {e}")
            continue
        bound = _bound_names(tree)
        for node in ast.walk(tree):
            if isinstance(node, ast.Name) and isinstance(node.ctx, ast.Load) and node.id not in bound:
                problems.append(f"{os.path.relpath(path, ROOT)}:{node.lineno}: name '{node.id}' is never bound in this file")
    assert not problems, "\n".join(problems)


def test_bench_reference_arm_answers_without_a_gpu():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "--schedule" in r.stdout and "--gpus" in r.stdout


def test_packaging_lists_every_subpackage_and_the_package_version():
    out = subprocess.run([sys.executable, "setup.py", "--version"], cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    scope = {}
    exec(open(os.path.join(ROOT, "moodist_b200", "version.py")).read(), scope)
    assert out.stdout.strip().splitlines()[-1] == scope["__version__"]
    # every directory of the package that holds an __init__.py is named in setup.py (a new one is easy to forget)
    src = open(os.path.join(ROOT, "setup.py")).read()
    pkg = os.path.join(ROOT, "moodist_b200")
    for d, _, files in os.walk(pkg):
        if "__init__.py" in files:
            name = os.path.relpath(d, ROOT).replace(os.sep, ".")
            assert f'"{name}"' in src, f"{name} is missing from setup.py's package list"


def test_every_environment_variable_the_sources_read_is_documented():
    import re

    used = set()
    for top in ("moodist_b200", "bench.py", "setup.py", "benchmarks"):
        path = os.path.join(ROOT, top)
        files = [path] if os.path.isfile(path) else [os.path.join(d, f) for d, _, fs in os.walk(path) for f in fs
                                                     if f.endswith((".py", ".cc", ".cu", ".h", ".cuh"))]
        for f in files:
            used.update(re.findall(r'"(MOODIST_[A-Z0-9_]+)"', open(f, errors="replace").read()))
    page = open(os.path.join(ROOT, "docs", "api", "environment.md")).read()
    missing = sorted(v for v in used if f"`{v}`" not in page)
    assert not missing, f"not in docs/api/environment.md: {missing}"
