"""Name → class registries for agents and environments, filled by decorators, and discovery of the modules that
hold decorated classes (tunix/experimental/rl/agentic/registry.py:29-257).

    @register_agent("diagnostic")        # or @register_agent() / bare @register_agent: the class name is the key
    class DiagnosticAgent: ...
    AGENT_REGISTRY.get("diagnostic")

`auto_discover_modules("pkg.agents", "./my_envs")` imports only the files whose source has a class decorated with
one of the registry decorators (found by parsing, not by importing), so that a configuration can name classes from
user code without that code being imported by hand and without importing unrelated, possibly heavy, modules."""
from __future__ import annotations

import ast
import contextlib
import importlib
import importlib.util
import os
import pkgutil
import sys
from typing import Any, Optional

_DECORATOR_NAMES = {"register_agent", "register_env", "AGENT_REGISTRY", "ENV_REGISTRY"}


class Registry:
    def __init__(self, name: str = "Registry"):
        self.name = name
        self._registry: dict = {}

    def _add(self, key: str, cls):
        if key in self._registry:
            raise KeyError(f"Key '{key}' is already registered in {self.name} for class '{self._registry[key].__name__}'.")
        self._registry[key] = cls
        return cls

    def register(self, name: Any = None):
        if isinstance(name, type):                           # bare decorator
            return self._add(name.__name__, name)
        return lambda cls: self._add(name if name is not None else cls.__name__, cls)

    def get(self, name: str):
        try:
            return self._registry[name]
        except KeyError:
            raise KeyError(f"'{name}' is not registered in {self.name}. Available keys: {list(self._registry)}") from None

    def contains(self, name: str) -> bool:
        return name in self._registry

    __contains__ = contains

    def keys(self) -> list:
        return list(self._registry)


AGENT_REGISTRY = Registry("AgentRegistry")
ENV_REGISTRY = Registry("EnvRegistry")
register_agent = AGENT_REGISTRY.register
register_env = ENV_REGISTRY.register


def _dotted(node) -> list:
    """['a', 'b', 'c'] for the expression a.b.c (through a call: a.b.c(...))."""
    if isinstance(node, ast.Call):
        node = node.func
    parts = []
    while isinstance(node, ast.Attribute):
        parts.append(node.attr)
        node = node.value
    if isinstance(node, ast.Name):
        parts.append(node.id)
    return parts[::-1]


def has_registry_decorator(file_path: str) -> bool:
    """True when a class in the file is decorated with a registry decorator: one of the names above (also under an
    `import ... as` alias), `<registry>.register`, or `register` of a name bound to a `Registry(...)` in the file."""
    try:
        with open(file_path, encoding="utf-8") as f:
            tree = ast.parse(f.read(), filename=file_path)
    except Exception:
        return False
    names = set(_DECORATOR_NAMES)
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom):
            for a in node.names:
                if a.name in _DECORATOR_NAMES or (a.name in ("registry", "register") and (node.level or "agentic" in (node.module or ""))):
                    names.add(a.asname or a.name)
        elif isinstance(node, ast.Import):
            for a in node.names:
                if "agentic" in a.name and "registry" in a.name:
                    names.add((a.asname or a.name).split(".")[-1] if a.asname else a.name.split(".")[-1])
        elif isinstance(node, ast.Assign):
            src = _dotted(node.value)
            if src and (src[-1] in names or src[-1] == "Registry" or (src[-1] == "register" and len(src) > 1 and src[-2] in names)):
                names.update(t.id for t in node.targets if isinstance(t, ast.Name))
    for node in ast.walk(tree):
        if isinstance(node, ast.ClassDef):
            for dec in node.decorator_list:
                parts = _dotted(dec)
                if parts and (parts[-1] in names or (parts[-1] == "register" and any(p in names for p in parts[:-1]))):
                    return True
    return False


def _module_name_of(file_path: str) -> Optional[str]:
    path = os.path.abspath(file_path)
    for entry in sys.path:
        if entry and path.startswith(os.path.abspath(entry) + os.sep):
            return os.path.splitext(os.path.relpath(path, os.path.abspath(entry)))[0].replace(os.sep, ".")
    return None


@contextlib.contextmanager
def _on_sys_path(directory: str):
    directory = os.path.abspath(directory)
    added = _module_name_of(os.path.join(directory, "x.py")) is None and directory not in sys.path
    if added:
        sys.path.insert(0, directory)
    try:
        yield directory
    finally:
        if added:
            with contextlib.suppress(ValueError):
                sys.path.remove(directory)


def auto_discover_modules(*package_or_directory_paths: str) -> list:
    """Import the modules under the given import paths or directories that hold decorated classes; returns their names."""
    imported = []
    for target in package_or_directory_paths:
        if os.path.isdir(target):
            with _on_sys_path(target) as root:
                for dirpath, _, files in os.walk(root):
                    for fn in sorted(files):
                        path = os.path.join(dirpath, fn)
                        if fn.endswith(".py") and not fn.startswith("__") and has_registry_decorator(path):
                            mod = _module_name_of(path)
                            if mod:
                                importlib.import_module(mod)
                                imported.append(mod)
            continue
        mod = importlib.import_module(target)
        if hasattr(mod, "__path__"):
            for _, sub, _ in pkgutil.walk_packages(mod.__path__, prefix=mod.__name__ + "."):
                try:
                    spec = importlib.util.find_spec(sub)
                    if spec and spec.origin and os.path.exists(spec.origin) and has_registry_decorator(spec.origin):
                        importlib.import_module(sub)
                        imported.append(sub)
                except Exception:                               # a broken sibling module does not stop discovery
                    pass
    return imported
