"""Hydra-style config composition and command-line overrides, without Hydra.

Implements the part of Hydra 1.3 that the reference's ``configs/`` tree and scripts rely on
(scripts/train.py:38-67 with ``@hydra.main``; configs/train/*.yaml):

* ``defaults:`` lists with ``_self_``, sibling files (``- defaults.yaml``), config groups
  (``- lr_scheduler: wsd``, nested ``- optimization/amp: bfloat16``), ``optional``, ``override``
  prefixes, ``group@package: option`` and ``group: null``; ``hydra/*`` groups are ignored.
* ``# @package _global_`` / ``# @package a.b`` headers.
* Overrides: ``a.b=v``, ``+a.b=v``, ``++a.b=v``, ``~a.b``, ``group=option``, ``group/sub=option``.
* ``--config-name/-cn``, ``--config-path/-cp``, ``--config-dir/-cd``, ``--cfg/-c job``, ``--multirun/-m``
  (comma sweeps expand to the cartesian product).
* ``hydra.job.env_set`` entries are exported to the environment; the ``hydra`` key is dropped.
"""

from __future__ import annotations

import functools
import itertools
import os
import re
import sys
from typing import Any, Callable

import yaml

from . import conf

_PKG_RE = re.compile(r"^#\s*@package\s+(\S+)\s*$", re.M)


class ComposeError(Exception):
    pass


def _read(path: str) -> tuple[dict, str | None]:
    with open(path) as f:
        text = f.read()
    m = _PKG_RE.search(text)
    data = yaml.safe_load(text)
    if data is None:
        data = {}
    if not isinstance(data, (dict, list)):
        raise ComposeError(f"{path}: top level must be a mapping or a list")
    pkg = m.group(1) if m else None
    if pkg is not None:
        pkg = pkg.lstrip("@")   # '# @package @_global_' is written in some configs; the package is _global_
    return data, pkg


def _find(config_dirs: list[str], rel: str) -> str | None:
    for d in config_dirs:
        for cand in (rel, rel + ".yaml", rel + ".yml"):
            p = os.path.join(d, cand)
            if os.path.isfile(p):
                return p
    return None


def _is_group(config_dirs: list[str], name: str) -> bool:
    return any(os.path.isdir(os.path.join(d, name)) for d in config_dirs)


def _place(content: dict, package: str | None) -> dict:
    if not package or package == "_global_":
        return content
    out: dict = {}
    cur = out
    parts = package.split(".")
    for p in parts[:-1]:
        cur = cur.setdefault(p, {})
    cur[parts[-1]] = content
    return out


def _parse_default(entry: Any) -> dict:
    """Normalise one defaults-list entry to {kind, group, option, package, optional, override}."""
    if isinstance(entry, str):
        if entry == "_self_":
            return {"kind": "self"}
        return {"kind": "file", "option": entry, "package": None, "optional": False}
    if isinstance(entry, dict) and len(entry) == 1:
        (k, v), = entry.items()
        k = str(k)
        optional = override = False
        while True:
            if k.startswith("optional "):
                optional, k = True, k[len("optional "):].strip()
            elif k.startswith("override "):
                override, k = True, k[len("override "):].strip()
            else:
                break
        package = None
        if "@" in k:
            k, package = k.split("@", 1)
        return {"kind": "group", "group": k.strip("/"), "option": v, "package": package, "optional": optional,
                "override": override}
    raise ComposeError(f"unsupported defaults entry: {entry!r}")


def _load_tree(config_dirs: list[str], rel: str, group_choices: dict[str, Any], parent_group: str = "") -> dict:
    """Load one config file and everything in its defaults list; returns a plain merged dict."""
    path = _find(config_dirs, rel)
    if path is None:
        raise ComposeError(f"config '{rel}' not found in {config_dirs}")
    data, header_pkg = _read(path)
    if isinstance(data, list):   # a group option may be a bare list (e.g. the loggers group)
        return data  # type: ignore[return-value]
    defaults = data.pop("defaults", None) or []
    if not any(d == "_self_" for d in defaults):
        defaults = list(defaults) + ["_self_"]
    merged = conf.create({})
    base_dir = os.path.dirname(rel)
    for entry in defaults:
        d = _parse_default(entry)
        if d["kind"] == "self":
            merged = conf.merge(merged, data)
            continue
        if d["kind"] == "file":
            sub_rel = os.path.join(base_dir, d["option"]) if base_dir else d["option"]
            if _find(config_dirs, sub_rel) is None and _find(config_dirs, d["option"]) is not None:
                sub_rel = d["option"]
            sub = _load_tree(config_dirs, sub_rel, group_choices, parent_group)
            merged = conf.merge(merged, sub)
            continue
        group = d["group"]
        if group.startswith("hydra/") or group == "hydra":
            continue
        if d["override"]:
            continue   # only changes the option of a group chosen elsewhere (collected by _collect_overrides)
        full_group = group if not base_dir or group.startswith("/") else group
        option = group_choices.get(full_group, d["option"])
        if option is None or option == "null":
            continue
        options = option if isinstance(option, list) else [option]
        for opt in options:
            sub_rel = os.path.join(base_dir, full_group, str(opt)) if base_dir and _find(config_dirs, os.path.join(base_dir, full_group, str(opt))) else os.path.join(full_group, str(opt))
            if _find(config_dirs, sub_rel) is None:
                if d["optional"]:
                    continue
                raise ComposeError(f"config group option '{full_group}/{opt}' not found in {config_dirs}")
            sub_path = _find(config_dirs, sub_rel)
            _, sub_header = _read(sub_path)
            sub = _load_tree(config_dirs, sub_rel, group_choices, full_group)
            pkg = d["package"] or sub_header
            if pkg is None:
                pkg = full_group.replace("/", ".")
            elif pkg == "_group_":
                pkg = full_group.replace("/", ".")
            sub_plain = conf.to_container(sub, resolve=False)
            # the file's own header was already applied by the recursive call only for _global_/explicit
            merged = conf.merge(merged, _place(sub_plain, None if sub_header else pkg))
    out = conf.to_container(merged, resolve=False)
    return _place(out, header_pkg) if header_pkg and header_pkg != "_global_" else out


def _collect_overrides(config_dirs: list[str], rel: str, out: dict[str, Any]) -> None:
    """``- override group: option`` entries of a config (and of the config files it includes) re-select the
    option of a group that some other defaults list chooses. The outermost file wins."""
    path = _find(config_dirs, rel)
    if path is None:
        return
    data, _ = _read(path)
    if not isinstance(data, dict):
        return
    base_dir = os.path.dirname(rel)
    for entry in data.get("defaults") or []:
        d = _parse_default(entry)
        if d["kind"] == "group" and d["override"] and not d["group"].startswith("hydra"):
            out.setdefault(d["group"], d["option"])
        elif d["kind"] == "file":
            sub_rel = os.path.join(base_dir, d["option"]) if base_dir else d["option"]
            if _find(config_dirs, sub_rel) is None:
                sub_rel = d["option"]
            _collect_overrides(config_dirs, sub_rel, out)


_OVR = re.compile(r"^(?P<prefix>\+\+|\+|~)?(?P<key>[^=]+?)(=(?P<value>.*))?$", re.S)


def parse_override(text: str) -> dict:
    m = _OVR.match(text)
    if not m:
        raise ComposeError(f"cannot parse override {text!r}")
    prefix, key, value = m.group("prefix") or "", m.group("key").strip(), m.group("value")
    if prefix == "~":
        return {"op": "delete", "key": key, "value": None if value is None else _parse_value(value)}
    if value is None:
        raise ComposeError(f"override {text!r} has no value")
    return {"op": {"": "set", "+": "add", "++": "force"}[prefix], "key": key, "value": _parse_value(value), "raw": value}


def _parse_value(v: str) -> Any:
    v = v.strip()
    if v == "":
        return ""
    try:
        return yaml.safe_load(v)
    except yaml.YAMLError:
        return v


def compose(config_dir: str | list[str], config_name: str, overrides: list[str] | None = None,
            apply_env: bool = True) -> conf.DictNode:
    """Compose ``config_name`` from ``config_dir`` and apply ``overrides``; returns the root node."""
    config_dirs = [config_dir] if isinstance(config_dir, str) else list(config_dir)
    config_dirs = [os.path.abspath(d) for d in config_dirs]
    parsed = [parse_override(o) for o in (overrides or [])]
    group_choices: dict[str, Any] = {}
    value_ops = []
    for o in parsed:
        gkey = o["key"].replace(".", "/") if _is_group(config_dirs, o["key"].replace(".", "/")) else o["key"]
        if o["op"] in ("set", "add", "force") and _is_group(config_dirs, gkey) and isinstance(o["value"], (str, list)) \
                and not isinstance(o["value"], dict):
            group_choices[gkey] = o["value"]
        elif o["op"] == "delete" and _is_group(config_dirs, gkey):
            group_choices[gkey] = None
        else:
            value_ops.append(o)
    file_overrides: dict[str, Any] = {}
    _collect_overrides(config_dirs, config_name, file_overrides)
    for g, opt in file_overrides.items():
        group_choices.setdefault(g, opt)   # the command line has priority
    plain = _load_tree(config_dirs, config_name, group_choices)
    # groups chosen on the command line that the defaults list did not mention are appended
    cfg = conf.create(plain)
    for g, opt in group_choices.items():
        if opt is None:
            continue
        if conf.select(cfg, g.replace("/", "."), default=None) is None:
            for o in (opt if isinstance(opt, list) else [opt]):
                rel = os.path.join(g, str(o))
                if _find(config_dirs, rel) is None:
                    raise ComposeError(f"config group option '{rel}' not found")
                sub = _load_tree(config_dirs, rel, group_choices, g)
                _, hdr = _read(_find(config_dirs, rel))
                cfg = conf.merge(cfg, _place(sub, None if hdr else g.replace("/", ".")))
    for o in value_ops:
        if o["op"] == "delete":
            try:
                conf.delete(cfg, o["key"])
            except (KeyError, conf.ConfigError, IndexError):
                raise ComposeError(f"cannot delete '{o['key']}': key not in config") from None
        elif o["op"] == "set":
            exists = conf.select_relative(cfg, o["key"], throw=False, default=_SENTINEL, resolve=False) is not _SENTINEL
            if not exists:
                # Hydra would consult the structured schema here; keys that only exist as dataclass
                # defaults (e.g. common.use_gpu) are therefore accepted without the '+' prefix
                import logging

                logging.getLogger(__name__).debug("override adds new key %s", o["key"])
            conf.update(cfg, o["key"], o["value"], force_add=True)
        else:
            conf.update(cfg, o["key"], o["value"], force_add=True)
    hydra_cfg = cfg._data.pop("hydra", None)
    if apply_env and isinstance(hydra_cfg, conf.DictNode):
        env = (conf.to_container(hydra_cfg, resolve=False).get("job") or {}).get("env_set") or {}
        for k, v in env.items():
            os.environ.setdefault(str(k), str(v))
    return cfg


_SENTINEL = object()


def parse_cli(argv: list[str]) -> dict:
    """Split Hydra-style argv into options and overrides."""
    out: dict[str, Any] = {"config_name": None, "config_path": None, "config_dirs": [], "cfg": None, "multirun": False,
                           "overrides": [], "help": False}
    i = 0
    while i < len(argv):
        a = argv[i]

        def take(flag_len: int) -> str:
            nonlocal i
            if "=" in a:
                return a.split("=", 1)[1]
            i += 1
            if i >= len(argv):
                raise ComposeError(f"{a} needs a value")
            return argv[i]

        if a.startswith("--config-name") or a == "-cn" or a.startswith("-cn="):
            out["config_name"] = take(0)
        elif a.startswith("--config-path") or a == "-cp" or a.startswith("-cp="):
            out["config_path"] = take(0)
        elif a.startswith("--config-dir") or a == "-cd" or a.startswith("-cd="):
            out["config_dirs"].append(take(0))
        elif a.startswith("--cfg") or a == "-c" or a.startswith("-c="):
            out["cfg"] = take(0)
        elif a in ("--multirun", "-m"):
            out["multirun"] = True
        elif a in ("--help", "-h"):
            out["help"] = True
        elif a == "--resolve":
            out["resolve"] = True
        else:
            out["overrides"].append(a)
        i += 1
    return out


def expand_sweeps(overrides: list[str]) -> list[list[str]]:
    """``a=1,2 b=x`` -> ``[[a=1,b=x],[a=2,b=x]]`` (commas inside brackets/quotes are kept)."""
    axes = []
    for o in overrides:
        if "=" in o and not o.startswith("~"):
            k, v = o.split("=", 1)
            parts = conf._split_args(v)
            if len(parts) > 1 and not (v.startswith("[") or v.startswith("{")):
                axes.append([f"{k}={p}" for p in parts])
                continue
        axes.append([o])
    return [list(c) for c in itertools.product(*axes)]


def main(config_path: str | None = None, config_name: str | None = None, version_base: Any = None) -> Callable:
    """Decorator equivalent of ``hydra.main``: the wrapped function receives the composed config."""

    def deco(fn: Callable[[conf.DictNode], Any]) -> Callable[..., Any]:
        @functools.wraps(fn)
        def wrapper(cfg_passthrough: Any = None) -> Any:
            if cfg_passthrough is not None:
                return fn(cfg_passthrough)
            cli = parse_cli(sys.argv[1:])
            base = os.path.dirname(os.path.abspath(sys.modules[fn.__module__].__file__))
            cpath = cli["config_path"] or config_path or "."
            cdir = cpath if os.path.isabs(cpath) else os.path.normpath(os.path.join(base, cpath))
            dirs = [cdir] + cli["config_dirs"]
            name = cli["config_name"] or config_name
            if name is None:
                raise ComposeError("no config name given (use --config-name)")
            runs = expand_sweeps(cli["overrides"]) if cli["multirun"] else [cli["overrides"]]
            result = None
            for ovr in runs:
                cfg = compose(dirs, name, ovr)
                if cli["cfg"]:
                    print(conf.to_yaml(cfg, resolve=bool(cli.get("resolve"))))
                    continue
                result = fn(cfg)
            return result

        return wrapper

    return deco
