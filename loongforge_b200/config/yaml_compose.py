"""A small YAML composer with the subset of Hydra/OmegaConf semantics the model configs use.

The reference composes its model YAML files with Hydra (``defaults`` lists with ``@package``
targets, ``_self_`` ordering, ``${...}`` resolvers and ``key=value`` command-line overrides;
loongforge/train/parser.py:43-77,111-140). Hydra and OmegaConf are not dependencies here: this module
implements exactly those features so that files written in the same schema load unchanged.

Supported:
  * ``defaults: [ "<rel/dir>@<dotted.package>: <name>", ..., _self_ ]`` (path relative to the file);
  * interpolation ``${oc.env:VAR[,default]}``, ``${act:gelu}``, ``${position_func:mrope_ids}``,
    ``${loss_func:default}``, ``${moe_freq:...}`` and plain ``${a.b.c}`` references;
  * overrides ``a.b=1``, ``+a.b=1`` (add), ``~a.b`` (delete); values are parsed as YAML scalars.
"""
from __future__ import annotations

import ast
import copy
import os
import re
from typing import Any, Callable, Dict, List, Optional

import yaml

_RESOLVERS: Dict[str, Callable[..., Any]] = {}


def register_resolver(name: str, fn: Callable[..., Any]) -> None:
    _RESOLVERS[name] = fn


def _env(var: str, default: Optional[str] = None):
    v = os.environ.get(var.strip())
    if v is None:
        if default is None:
            if var.strip() == "LOONGFORGE_PATH":
                return os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            raise KeyError(f"environment variable {var} is not set and has no default")
        return default.strip()
    return v


def _moe_freq(expr: str):
    """``${moe_freq:([0]*3+[1]*58)}`` style python list expressions, or an integer."""
    val = ast.literal_eval(expr) if re.fullmatch(r"[\d\s]+", expr) else eval(expr, {"__builtins__": {}}, {})  # noqa: S307
    return val


register_resolver("oc.env", _env)
register_resolver("act", lambda name: str(name).strip())
register_resolver("position_func", lambda name: str(name).strip())
register_resolver("loss_func", lambda name: str(name).strip())
register_resolver("moe_freq", _moe_freq)

_INTERP = re.compile(r"\$\{([^${}]+)\}")


def _deep_merge(base: dict, other: dict) -> dict:
    for k, v in other.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _deep_merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _set_path(cfg: dict, dotted: str, value, create: bool = True):
    keys = dotted.split(".")
    cur = cfg
    for k in keys[:-1]:
        if k not in cur or not isinstance(cur[k], dict):
            if not create:
                raise KeyError(dotted)
            cur[k] = {}
        cur = cur[k]
    cur[keys[-1]] = value


def _get_path(cfg: dict, dotted: str):
    cur = cfg
    for k in dotted.split("."):
        cur = cur[k]
    return cur


def _del_path(cfg: dict, dotted: str):
    keys = dotted.split(".")
    cur = cfg
    for k in keys[:-1]:
        cur = cur[k]
    cur.pop(keys[-1], None)


def _load_file(path: str) -> dict:
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ValueError(f"{path}: top level must be a mapping")
    return data


def _compose_file(path: str, seen: Optional[List[str]] = None) -> dict:
    path = os.path.abspath(path)
    seen = (seen or []) + [path]
    data = _load_file(path)
    defaults = data.pop("defaults", None)
    if not defaults:
        return data
    out: dict = {}
    self_done = False
    base_dir = os.path.dirname(path)
    for entry in defaults:
        if entry == "_self_":
            _deep_merge(out, data)
            self_done = True
            continue
        if isinstance(entry, dict):
            (k, name), = entry.items()
        else:
            k, name = str(entry), None
        group, _, package = k.partition("@")
        if name is None:
            group, name = os.path.dirname(group), os.path.basename(group)
        sub_path = os.path.normpath(os.path.join(base_dir, group, str(name)))
        if not sub_path.endswith((".yaml", ".yml")):
            sub_path += ".yaml"
        if sub_path in seen:
            raise ValueError(f"cyclic defaults: {sub_path}")
        sub = _compose_file(sub_path, seen)
        if package:
            wrapped: dict = {}
            _set_path(wrapped, package, sub)
            sub = wrapped
        _deep_merge(out, sub)
    if not self_done:
        _deep_merge(out, data)
    return out


def _resolve_value(v, root: dict, depth: int = 0):
    if depth > 16:
        raise ValueError("interpolation nesting too deep")
    if isinstance(v, dict):
        return {k: _resolve_value(x, root, depth) for k, x in v.items()}
    if isinstance(v, list):
        return [_resolve_value(x, root, depth) for x in v]
    if not isinstance(v, str) or "${" not in v:
        return v

    def one(expr: str):
        name, sep, arg = expr.partition(":")
        if sep and name in _RESOLVERS:
            args = [a for a in arg.split(",")] if name == "oc.env" else [arg]
            return _RESOLVERS[name](*args)
        return _resolve_value(_get_path(root, expr.strip()), root, depth + 1)

    m = _INTERP.fullmatch(v)
    if m:  # whole value is one interpolation: keep the resolved type
        return one(m.group(1))
    return _INTERP.sub(lambda mm: str(one(mm.group(1))), v)


def parse_override(token: str):
    """'a.b=1' -> ('set', 'a.b', 1); '+a.b=x' -> ('add', ...); '~a.b' -> ('del', 'a.b', None)."""
    if token.startswith("~"):
        return "del", token[1:].split("=")[0], None
    op = "set"
    if token.startswith("++"):
        token = token[2:]
        op = "add"
    elif token.startswith("+"):
        token = token[1:]
        op = "add"
    key, sep, val = token.partition("=")
    if not sep:
        raise ValueError(f"override {token!r} is not of the form key=value")
    return op, key.strip(), yaml.safe_load(val) if val != "" else None


def compose(path: str, overrides: Optional[List[str]] = None, resolve: bool = True) -> dict:
    """Load `path`, apply its defaults list, the overrides, then resolve interpolations."""
    cfg = _compose_file(path)
    for tok in overrides or []:
        op, key, val = parse_override(tok)
        if op == "del":
            _del_path(cfg, key)
        else:
            if op == "set":
                try:
                    _get_path(cfg, key)
                except (KeyError, TypeError):
                    raise KeyError(f"override {tok!r}: key does not exist (use +{key}=... to add it)") from None
            _set_path(cfg, key, val)
    return _resolve_value(cfg, cfg) if resolve else cfg


def is_override_token(tok: str) -> bool:
    return bool(re.match(r"^(\+\+?|~)?[A-Za-z_][\w.]*(=.*)?$", tok)) and ("=" in tok or tok.startswith("~"))
