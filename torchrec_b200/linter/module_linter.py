"""Docstring linter for ``nn.Module`` subclasses (``torchrec/linter/module_linter.py``): every public module class documents what
it does, its constructor arguments, an example and its ``forward`` arguments and return value.  Findings are printed as JSON
lines (path, line, name, description) so that a review tool can attach them to the source.

    python -m torchrec_b200.linter.module_linter file1.py file2.py
"""
from __future__ import annotations

import ast
import json
import sys
from argparse import ArgumentParser, Namespace
from typing import Any, Dict, List, Optional, Tuple

MAX_NUM_ARGS_IN_MODULE_CTOR = 5


def print_error_message(python_path: str, node: ast.AST, name: str, message: str, severity: str = "warning") -> None:
    print(json.dumps({"path": python_path, "line": getattr(node, "lineno", 0), "char": getattr(node, "col_offset", 0), "severity": severity,
                      "name": name, "description": message}))


def get_function_args(node: ast.FunctionDef) -> Tuple[List[Any], List[Any]]:
    """``(argument names without self, argument names that have a default)``."""
    assert isinstance(node, ast.FunctionDef) and node.args.args and node.args.args[0].arg == "self", "expected a method"
    names = [a.arg for a in node.args.args[1:]] + [a.arg for a in node.args.kwonlyargs]
    n_def = len(node.args.defaults)
    with_default = [a.arg for a in node.args.args[len(node.args.args) - n_def:]] if n_def else []
    with_default += [a.arg for a, d in zip(node.args.kwonlyargs, node.args.kw_defaults) if d is not None]
    return names, with_default


def _is_module_class(node: ast.ClassDef) -> bool:
    for b in node.bases:
        if (isinstance(b, ast.Attribute) and b.attr == "Module") or (isinstance(b, ast.Name) and b.id == "Module"):
            return True
    return False


def check_class_definition(python_path: str, node: ast.ClassDef) -> None:
    if not _is_module_class(node) or node.name.startswith("_"):
        return
    doc = ast.get_docstring(node)
    if doc is None:
        print_error_message(python_path, node, "No docstring found in a module class", "Module classes need a docstring: what it does, Args:, Example::")
        return
    functions: Dict[str, Tuple[List[Any], List[Any]]] = {}
    fn_nodes: Dict[str, ast.FunctionDef] = {}
    for sub in node.body:
        if isinstance(sub, ast.FunctionDef):
            fn_nodes[sub.name] = sub
            try:
                functions[sub.name] = get_function_args(sub)
            except AssertionError:
                pass

    def check_function(function_name: str) -> None:
        if function_name not in functions:
            return
        names, with_default = functions[function_name]
        where = doc if function_name == "__init__" else (ast.get_docstring(fn_nodes[function_name]) or "")
        if function_name == "__init__" and len(names) > MAX_NUM_ARGS_IN_MODULE_CTOR and len(with_default) < len(names) - MAX_NUM_ARGS_IN_MODULE_CTOR:
            print_error_message(python_path, node, "Too many required constructor arguments",
                                f"{node.name}.__init__ has {len(names)} arguments, more than {MAX_NUM_ARGS_IN_MODULE_CTOR} of them required: give defaults or group them")
        if names and "Args:" not in where:
            print_error_message(python_path, fn_nodes[function_name], f"Missing Args: section for {function_name}", f"document the arguments of {node.name}.{function_name}")
            return
        for a in names:
            if a not in where:
                print_error_message(python_path, fn_nodes[function_name], f"Undocumented argument {a}", f"{node.name}.{function_name}: argument `{a}` is not described")

    check_function("__init__")
    if "forward" in fn_nodes:
        fdoc = ast.get_docstring(fn_nodes["forward"])
        if fdoc is None:
            print_error_message(python_path, fn_nodes["forward"], "No docstring on forward", f"{node.name}.forward needs Args: and Returns:")
        else:
            check_function("forward")
            if "Returns:" not in fdoc:
                print_error_message(python_path, fn_nodes["forward"], "Missing Returns: section", f"{node.name}.forward does not describe what it returns")
    if "Example" not in doc:
        print_error_message(python_path, node, "No runnable example", f"{node.name}: add an `Example::` block to the class docstring")


def read_file(path: str) -> str:  # pragma: nocover
    with open(path) as f:
        return f.read()


def linter_one_file(python_path: str) -> None:
    base = python_path.rsplit("/", 1)[-1]
    if "/tests/" in python_path or base.startswith("test_") or base.endswith("_test.py"):
        return
    try:
        tree = ast.parse(read_file(python_path))
    except SyntaxError as e:  # pragma: nocover
        print_error_message(python_path, ast.Module(body=[], type_ignores=[]), "Syntax error", str(e), "error")
        return
    for node in ast.walk(tree):
        if isinstance(node, ast.ClassDef):
            check_class_definition(python_path, node)


def _make_argparse() -> ArgumentParser:  # pragma: nocover
    p = ArgumentParser(description="docstring linter for module classes", fromfile_prefix_chars="@")
    p.add_argument("source_files", nargs="+", help="paths of the python files to lint")
    return p


def _parse_args() -> Namespace:  # pragma: nocover
    return _make_argparse().parse_args()


if __name__ == "__main__":  # pragma: nocover
    for path in _parse_args().source_files:
        linter_one_file(path)
