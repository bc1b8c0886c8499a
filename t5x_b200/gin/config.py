"""A gin-config compatible configuration system (the subset the T5X config corpus uses).

Supported syntax: comments, `from __gin__ import dynamic_registration`, `import a.b [as c]`,
`from a import b [as c]`, `include 'path'` (with search paths), macros `NAME = value` /
`%NAME` / `%gin.REQUIRED`, bindings `scope/.../module.fn.arg = value` and the block form
`module.fn:` + indented `arg = value`, references `@fn` (the configured callable) and `@fn()`
(its result, evaluated each time it is injected), scoped references `@train/utils.Cfg()`,
Python literals (dict / list / tuple / str / number / None / bool, implicit string
concatenation), later bindings overriding earlier ones, and method bindings
(`Class.method.arg = value`).

With dynamic registration a dotted name is resolved through the file's imports to any Python
callable; module names of the reference project (`t5x.*`, `seqio`) are aliased to this
package, so its `.gin` files load unmodified.
"""
from __future__ import annotations

import contextlib
import functools
import importlib
import inspect
import logging
import os
import re
import threading
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

# ----------------------------------------------------------------------------
# Module aliases: names used by the reference's gin files -> modules of this package
# ----------------------------------------------------------------------------
MODULE_ALIASES = {
    "t5x": "t5x_b200",
    "t5x.examples.t5.network": "t5x_b200.models.t5.network",
    "t5x.examples.t5.layers": "t5x_b200.models.t5.layers",
    "t5x.examples.t5": "t5x_b200.models.t5",
    "t5x.examples.scalable_t5.network": "t5x_b200.models.scalable_t5.network",
    "t5x.examples.scalable_t5.layers": "t5x_b200.models.scalable_t5.layers",
    "t5x.examples.scalable_t5": "t5x_b200.models.scalable_t5",
    "t5x.examples.decoder_only.network": "t5x_b200.models.decoder_only.network",
    "t5x.examples.decoder_only.layers": "t5x_b200.models.decoder_only.layers",
    "t5x.examples.decoder_only": "t5x_b200.models.decoder_only",
    "t5x.contrib.gpu.t5.network": "t5x_b200.models.t5.network",
    "t5x.contrib.gpu.t5.layers": "t5x_b200.models.t5.layers",
    "t5x.contrib.moe": "t5x_b200.contrib.moe",
    "t5x.contrib.calm": "t5x_b200.contrib.calm",
    "seqio": "t5x_b200.data.seqio_api",
    "optax": "t5x_b200.optax_api",
}
# Imports that only register datasets / are unavailable offline: ignored when missing.
OPTIONAL_IMPORT_PREFIXES = ("t5.", "t5", "tensorflow", "tensorflow_datasets", "flaxformer",
                            "t5x.contrib.gpu.scripts_gpu", "google", "jax", "flax", "clu", "tfds",
                            "t5x.google", "fiddle")


class _Required:
  def __repr__(self):
    return "%gin.REQUIRED"


REQUIRED = _Required()


class GinError(Exception):
  pass


# ----------------------------------------------------------------------------
# Values
# ----------------------------------------------------------------------------
class ConfigurableReference:
  """`@scope/name` or `@scope/name()`."""

  def __init__(self, name: str, scope: str, evaluate: bool, imports: Dict[str, Any]):
    self.name = name
    self.scope = scope
    self.evaluate = evaluate
    self._imports = imports

  def resolve(self):
    target = _resolve_name(self.name, self._imports)
    fn = _configured_callable(target, self.name, self.scope)
    return fn() if self.evaluate else fn

  def __repr__(self):
    s = "@" + (self.scope + "/" if self.scope else "") + self.name
    return s + ("()" if self.evaluate else "")


class MacroReference:
  def __init__(self, name: str):
    self.name = name

  def resolve(self):
    if self.name == "gin.REQUIRED":
      return REQUIRED
    key = ("", "macro", self.name)
    if key not in _CONFIG:
      raise GinError(f"Macro %{self.name} is not defined")
    return _materialize(_CONFIG[key])

  def __repr__(self):
    return "%" + self.name


def _materialize(v):
  """Evaluates references / macros inside a parsed value."""
  if isinstance(v, (ConfigurableReference, MacroReference)):
    return v.resolve()
  if isinstance(v, list):
    return [_materialize(x) for x in v]
  if isinstance(v, tuple):
    return tuple(_materialize(x) for x in v)
  if isinstance(v, dict):
    return {_materialize(k): _materialize(x) for k, x in v.items()}
  return v


def _format_value(v) -> str:
  if isinstance(v, (ConfigurableReference, MacroReference, _Required)):
    return repr(v)
  if isinstance(v, list):
    return "[" + ", ".join(_format_value(x) for x in v) + "]"
  if isinstance(v, tuple):
    return "(" + ", ".join(_format_value(x) for x in v) + ("," if len(v) == 1 else "") + ")"
  if isinstance(v, dict):
    return "{" + ", ".join(f"{_format_value(k)}: {_format_value(x)}" for k, x in v.items()) + "}"
  return repr(v)


# ----------------------------------------------------------------------------
# Global state
# ----------------------------------------------------------------------------
# (scope, selector, param) -> value.   selector "macro" holds macros.
_CONFIG: Dict[Tuple[str, str, str], Any] = {}
_OPERATIVE: Dict[Tuple[str, str, str], Any] = {}
_REGISTRY: Dict[str, Any] = {}       # explicitly registered configurables by name
_SELECTOR_OF: Dict[int, List[str]] = {}  # id(callable) -> selectors it was bound under
_SEARCH_PATHS: List[str] = []
_IMPORTS: Dict[str, Any] = {}        # alias -> module (accumulated over all parsed files)
_ACTIVE_SCOPES = threading.local()
_FINALIZED = False
_PATCHED_METHODS: Dict[Tuple[int, str], Any] = {}
_LOCK = threading.RLock()


def clear_config(clear_constants: bool = False) -> None:
  global _FINALIZED
  _CONFIG.clear()
  _OPERATIVE.clear()
  _SELECTOR_OF.clear()
  _IMPORTS.clear()
  _FINALIZED = False


def add_config_file_search_path(path: str) -> None:
  if path not in _SEARCH_PATHS:
    _SEARCH_PATHS.append(path)


def _scopes() -> List[str]:
  return getattr(_ACTIVE_SCOPES, "stack", [])


@contextlib.contextmanager
def config_scope(name: Optional[str]):
  stack = list(_scopes())
  new = stack + ([s for s in name.split("/") if s] if name else [])
  _ACTIVE_SCOPES.stack = new
  try:
    yield
  finally:
    _ACTIVE_SCOPES.stack = stack


# ----------------------------------------------------------------------------
# Name resolution
# ----------------------------------------------------------------------------
def _import_module(name: str):
  real = name
  for src in sorted(MODULE_ALIASES, key=len, reverse=True):
    if name == src or name.startswith(src + "."):
      real = MODULE_ALIASES[src] + name[len(src):]
      break
  return importlib.import_module(real)


def _resolve_name(name: str, imports: Dict[str, Any]):
  """`alias.attr[.attr]`, a registered name, or a fully qualified dotted path."""
  if name in _REGISTRY:
    return _REGISTRY[name]
  parts = name.split(".")
  # registered under "module.name" suffix
  for reg, obj in _REGISTRY.items():
    if reg.split(".")[-len(parts):] == parts:
      return obj
  scope_imports = dict(_IMPORTS)
  scope_imports.update(imports or {})
  for n in range(len(parts), 0, -1):
    head = ".".join(parts[:n])
    obj = scope_imports.get(head)
    if obj is None and n == len(parts):
      continue
    if obj is None:
      continue
    try:
      for attr in parts[n:]:
        obj = getattr(obj, attr)
      return obj
    except AttributeError:
      continue
  for n in range(len(parts) - 1, 0, -1):
    try:
      obj = _import_module(".".join(parts[:n]))
    except ImportError:
      continue
    try:
      for attr in parts[n:]:
        obj = getattr(obj, attr)
      return obj
    except AttributeError:
      continue
  raise GinError(f"Could not resolve configurable '{name}'")


def _selector_matches(selector: str, name: str) -> bool:
  """A binding selector matches a reference name if one is a dotted suffix of the other."""
  a, b = selector.split("."), name.split(".")
  n = min(len(a), len(b))
  return a[-n:] == b[-n:]


def _canonical(obj) -> str:
  mod = getattr(obj, "__module__", None) or ""
  qual = getattr(obj, "__qualname__", None) or getattr(obj, "__name__", repr(obj))
  return f"{mod}.{qual}"


def _bindings_for(target, name: str, scope: str) -> Dict[str, Any]:
  """Bindings that apply to `target` under the active scopes (outer scopes first)."""
  scopes = _scopes() + ([s for s in scope.split("/") if s] if scope else [])
  canon = _canonical(target)
  selectors = set(_SELECTOR_OF.get(id(target), []))
  out: Dict[str, Any] = {}
  prefixes = [""] + ["/".join(scopes[:i + 1]) for i in range(len(scopes))]
  # also individual scope names (gin matches any suffix of the active scope chain)
  for i in range(len(scopes)):
    prefixes.append("/".join(scopes[i:]))
  seen = []
  for p in prefixes:
    if p in seen:
      continue
    seen.append(p)
    for (sc, sel, param), val in _CONFIG.items():
      if sc != p or sel == "macro":
        continue
      if sel in selectors or _selector_matches(sel, canon) or (name and _selector_matches(sel, name)
                                                               and sel.split(".")[-1] == name.split(".")[-1]):
        out[param] = ((sc, sel, param), val)
  return out


def _configured_callable(target, name: str = "", scope: str = ""):
  """A callable that injects the bound parameters into `target` when called."""
  if not callable(target):
    raise GinError(f"'{name}' resolved to a non-callable {type(target)}")
  outer_scopes = list(_scopes())

  @functools.wraps(target, updated=())
  def call(*args, **kwargs):
    saved = list(_scopes())
    _ACTIVE_SCOPES.stack = outer_scopes if not saved else saved
    try:
      bound = _bindings_for(target, name, scope)
      try:
        sig = inspect.signature(target)
        params = sig.parameters
        positional = [p for p in params.values()
                      if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        passed = {p.name for p in positional[:len(args)]}
        accepts_kwargs = any(p.kind == p.VAR_KEYWORD for p in params.values())
      except (TypeError, ValueError):
        params, passed, accepts_kwargs = {}, set(), True
      inject = {}
      with config_scope(scope):
        for pname, (key, val) in bound.items():
          if pname in kwargs or pname in passed:
            continue
          if params and pname not in params and not accepts_kwargs:
            raise GinError(f"'{name or _canonical(target)}' has no parameter '{pname}' "
                           f"(bound in the config)")
          v = _materialize(val)
          if v is REQUIRED:
            raise GinError(f"Required binding for '{name or _canonical(target)}.{pname}' "
                           "was not provided")
          inject[pname] = v
          _OPERATIVE[key] = val
        return target(*args, **inject, **kwargs)
    finally:
      _ACTIVE_SCOPES.stack = saved

  call.__gin_target__ = target
  return call


def get_configurable(fn_or_name):
  """The gin-configured version of a callable (or of a registered name)."""
  if isinstance(fn_or_name, str):
    return _configured_callable(_resolve_name(fn_or_name, _IMPORTS), fn_or_name)
  return _configured_callable(fn_or_name, getattr(fn_or_name, "__name__", ""))


def configurable(name_or_fn=None, module: Optional[str] = None, allowlist=None, denylist=None,
                 **_):
  """Decorator: calls of the decorated function / class constructor receive bound
  parameters that the caller did not pass."""

  def decorate(obj, name=None):
    reg_name = name or obj.__name__
    if inspect.isclass(obj):
      orig_init = obj.__init__

      @functools.wraps(orig_init)
      def init(self, *args, **kwargs):
        bound = _bindings_for(obj, reg_name, "")
        try:
          params = inspect.signature(orig_init).parameters
        except (TypeError, ValueError):
          params = {}
        positional = [p for p in list(params.values())[1:]
                      if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        passed = {p.name for p in positional[:len(args)]}
        for pname, (key, val) in bound.items():
          if pname in kwargs or pname in passed or (params and pname not in params):
            continue
          v = _materialize(val)
          if v is not REQUIRED:
            kwargs[pname] = v
            _OPERATIVE[key] = val
        orig_init(self, *args, **kwargs)

      obj.__init__ = init
      wrapped = obj
    else:
      wrapped = _configured_callable(obj, reg_name)
    full = f"{module}.{reg_name}" if module else reg_name
    _REGISTRY[full] = obj
    _SELECTOR_OF.setdefault(id(obj), []).append(full)
    return wrapped

  if callable(name_or_fn) and not isinstance(name_or_fn, str):
    return decorate(name_or_fn)
  return lambda obj: decorate(obj, name_or_fn)


def register(name_or_fn=None, module: Optional[str] = None, **kw):
  """Registers a callable under a name without changing its direct-call behaviour."""

  def decorate(obj, name=None):
    reg_name = name or obj.__name__
    _REGISTRY[f"{module}.{reg_name}" if module else reg_name] = obj
    return obj

  if callable(name_or_fn) and not isinstance(name_or_fn, str):
    return decorate(name_or_fn)
  return lambda obj: decorate(obj, name_or_fn)


external_configurable = lambda fn, name=None, module=None, **_: register(name, module)(fn) \
    if name else register(fn, module=module)


def constant(name: str, value) -> None:
  _CONFIG[("", "macro", name)] = value


def bind_parameter(binding_key: str, value) -> None:
  scope, selector, param = _split_binding_key(binding_key)
  _CONFIG[(scope, selector, param)] = value


def query_parameter(binding_key: str):
  if binding_key.startswith("%"):
    return _CONFIG[("", "macro", binding_key[1:])]
  scope, selector, param = _split_binding_key(binding_key)
  if selector == "macro" or (not selector and ("", "macro", param) in _CONFIG):
    return _CONFIG[("", "macro", param)]
  for (sc, sel, p), v in _CONFIG.items():
    if sc == scope and p == param and (_selector_matches(sel, selector)):
      return v
  raise ValueError(f"Configurable '{selector}' has no bound parameter '{param}'")


def _split_binding_key(key: str):
  scope = ""
  if "/" in key:
    scope, key = key.rsplit("/", 1)
  if "." not in key:
    return scope, "macro", key
  selector, param = key.rsplit(".", 1)
  return scope, selector, param


# ----------------------------------------------------------------------------
# Value parser
# ----------------------------------------------------------------------------
_TOKEN = re.compile(r"""
    (?P<ws>\s+)
  | (?P<str>(?:[rRbBuU]{0,2})(?:'''(?:\\.|[^\\])*?'''|\"\"\"(?:\\.|[^\\])*?\"\"\"|'(?:\\.|[^'\\\n])*'|"(?:\\.|[^"\\\n])*"))
  | (?P<num>[+-]?(?:0[xX][0-9a-fA-F]+|(?:\d[\d_]*\.[\d_]*|\.\d[\d_]*|\d[\d_]*)(?:[eE][+-]?\d+)?j?))
  | (?P<ref>@[A-Za-z_][\w./]*(?:\(\))?)
  | (?P<macro>%[A-Za-z_][\w.]*)
  | (?P<name>[A-Za-z_][\w.]*)
  | (?P<punct>[\[\]{}(),:])
""", re.VERBOSE | re.DOTALL)


class _ValueParser:
  def __init__(self, text: str, imports: Dict[str, Any]):
    self.toks = []
    pos = 0
    while pos < len(text):
      m = _TOKEN.match(text, pos)
      if not m:
        raise GinError(f"Cannot parse value near: {text[pos:pos + 40]!r}")
      pos = m.end()
      if m.lastgroup != "ws":
        self.toks.append((m.lastgroup, m.group(m.lastgroup)))
    self.i = 0
    self.imports = imports

  def peek(self):
    return self.toks[self.i] if self.i < len(self.toks) else (None, None)

  def next(self):
    t = self.peek()
    self.i += 1
    return t

  def parse(self):
    v = self.value()
    if self.i != len(self.toks):
      raise GinError(f"Unexpected trailing tokens: {self.toks[self.i:]}")
    return v

  def value(self):
    kind, tok = self.next()
    if kind == "str":
      import ast
      s = ast.literal_eval(tok)
      while self.peek()[0] == "str":  # implicit concatenation
        s += ast.literal_eval(self.next()[1])
      return s
    if kind == "num":
      import ast
      return ast.literal_eval(tok)
    if kind == "ref":
      evaluate = tok.endswith("()")
      body = tok[1:-2] if evaluate else tok[1:]
      scope, name = ("", body)
      if "/" in body:
        scope, name = body.rsplit("/", 1)
      return ConfigurableReference(name, scope, evaluate, self.imports)
    if kind == "macro":
      return MacroReference(tok[1:])
    if kind == "name":
      if tok == "True":
        return True
      if tok == "False":
        return False
      if tok == "None":
        return None
      if tok in ("inf", "nan"):
        return float(tok)
      raise GinError(f"Unquoted name '{tok}' is not a valid gin value")
    if kind == "punct":
      if tok == "[":
        return self.sequence("]")
      if tok == "(":
        items, trailing = self.sequence(")", want_trailing=True)
        if len(items) == 1 and not trailing:
          return items[0]
        return tuple(items)
      if tok == "{":
        d = {}
        while True:
          if self.peek() == ("punct", "}"):
            self.next()
            return d
          k = self.value()
          if self.next() != ("punct", ":"):
            raise GinError("Expected ':' in dict")
          d[k] = self.value()
          if self.peek() == ("punct", ","):
            self.next()
    raise GinError(f"Unexpected token {tok!r}")

  def sequence(self, close, want_trailing=False):
    items = []
    trailing = False
    while True:
      if self.peek() == ("punct", close):
        self.next()
        return (items, trailing) if want_trailing else items
      items.append(self.value())
      trailing = False
      if self.peek() == ("punct", ","):
        self.next()
        trailing = True


def parse_value(text: str, imports: Optional[Dict[str, Any]] = None):
  return _ValueParser(text, imports if imports is not None else _IMPORTS).parse()


# ----------------------------------------------------------------------------
# File parser
# ----------------------------------------------------------------------------
def _strip_comment(line: str) -> str:
  out, quote, i = [], None, 0
  while i < len(line):
    c = line[i]
    if quote:
      out.append(c)
      if c == "\\" and i + 1 < len(line):
        out.append(line[i + 1])
        i += 1
      elif c == quote:
        quote = None
    elif c in "'\"":
      quote = c
      out.append(c)
    elif c == "#":
      break
    else:
      out.append(c)
    i += 1
  return "".join(out).rstrip()


def _balanced(text: str) -> bool:
  depth, quote, i = 0, None, 0
  triple = None
  while i < len(text):
    c = text[i]
    if triple:
      if text.startswith(triple, i):
        i += 3
        triple = None
        continue
    elif quote:
      if c == "\\":
        i += 1
      elif c == quote:
        quote = None
    elif text.startswith("'''", i) or text.startswith('"""', i):
      triple = text[i:i + 3]
      i += 3
      continue
    elif c in "'\"":
      quote = c
    elif c in "([{":
      depth += 1
    elif c in ")]}":
      depth -= 1
    i += 1
  return depth <= 0 and quote is None and triple is None


def _find_file(path: str, relative_to: Optional[str]) -> str:
  cands = [path]
  if relative_to:
    cands.append(os.path.join(os.path.dirname(relative_to), path))
  for sp in _SEARCH_PATHS:
    cands.append(os.path.join(sp, path))
    # reference configs are addressed as "t5x/...": also try them relative to our config root
    if path.startswith("t5x/"):
      cands.append(os.path.join(sp, path[len("t5x/"):]))
  for c in cands:
    if os.path.exists(c):
      return c
  raise GinError(f"Config file '{path}' not found; search paths: {_SEARCH_PATHS}")


def parse_config_file(path: str, skip_unknown: bool = False, _relative_to=None) -> None:
  real = _find_file(path, _relative_to)
  with open(real) as f:
    parse_config(f.read(), skip_unknown=skip_unknown, _filename=real)


_MAIN_MODULE = None


def set_main_module(module) -> None:
  """The object that `import __main__ as x` binds in config files. Entry points that are called
  as functions (rather than run as scripts) register themselves here."""
  global _MAIN_MODULE
  _MAIN_MODULE = module


def _do_import(stmt: str, imports: Dict[str, Any], skip_unknown: bool):
  m = re.match(r"from\s+([\w.]+)\s+import\s+(\w+)(?:\s+as\s+(\w+))?$", stmt)
  try:
    if m:
      mod, name, alias = m.groups()
      if mod == "__gin__":
        return
      try:
        obj = _import_module(f"{mod}.{name}")
      except ImportError:
        obj = getattr(_import_module(mod), name)
      imports[alias or name] = obj
      return
    m = re.match(r"import\s+([\w.]+)(?:\s+as\s+(\w+))?$", stmt)
    if not m:
      raise GinError(f"Cannot parse import statement: {stmt}")
    mod, alias = m.groups()
    if mod == "__main__":
      import sys
      obj = _MAIN_MODULE if _MAIN_MODULE is not None else sys.modules["__main__"]
    else:
      obj = _import_module(mod)
    if alias:
      imports[alias] = obj
    else:
      imports[mod] = obj
      imports.setdefault(mod.split(".")[0], _import_module(mod.split(".")[0]))
  except ImportError as e:
    target = stmt.split()[1]
    optional = any(target == p.rstrip(".") or target.startswith(p.rstrip(".") + ".")
                   for p in OPTIONAL_IMPORT_PREFIXES)
    if skip_unknown or optional:
      logging.info("gin: ignoring unavailable import '%s' (%s)", stmt, e)
      return
    raise


def parse_config(bindings, skip_unknown: bool = False, _filename: Optional[str] = None) -> None:
  """Parses gin statements from a string (or a list of binding strings)."""
  if isinstance(bindings, (list, tuple)):
    bindings = "\n".join(bindings)
  imports = _IMPORTS
  lines = bindings.split("\n")
  i = 0
  block_selector = None
  while i < len(lines):
    raw = lines[i]
    line = _strip_comment(raw)
    i += 1
    if not line.strip():
      continue
    indented = raw[:1] in (" ", "\t")
    if not indented:
      block_selector = None
    stmt = line.strip()
    # gather continuation lines: an open bracket or a trailing backslash
    while i < len(lines) and (stmt.endswith("\\") or not _balanced(stmt)):
      if stmt.endswith("\\"):
        stmt = stmt[:-1].rstrip() + " " + _strip_comment(lines[i]).strip()
      else:
        stmt += "\n" + _strip_comment(lines[i])
      i += 1
    if stmt.startswith("import ") or stmt.startswith("from "):
      _do_import(" ".join(stmt.split()), imports, skip_unknown)
      continue
    if stmt.startswith("include "):
      inc = parse_value(stmt[len("include "):].strip(), imports)
      parse_config_file(inc, skip_unknown=skip_unknown, _relative_to=_filename)
      continue
    if re.match(r"^[\w./]+:\s*$", stmt) and not indented:
      block_selector = stmt[:-1].strip()
      continue
    if "=" not in stmt:
      raise GinError(f"Cannot parse gin statement: {stmt!r}")
    lhs, rhs = stmt.split("=", 1)
    lhs, rhs = lhs.strip(), rhs.strip()
    if indented and block_selector:
      lhs = f"{block_selector}.{lhs}"
    value = parse_value(rhs, imports)
    scope, selector, param = _split_binding_key(lhs)
    if selector != "macro":
      _bind_selector(selector, imports, skip_unknown)
    _CONFIG[(scope, selector, param)] = value


def _bind_selector(selector: str, imports, skip_unknown: bool) -> None:
  """Resolves the selector now (errors surface at parse time) and handles method bindings."""
  try:
    target = _resolve_name(selector, imports)
  except GinError:
    if skip_unknown:
      return
    raise
  _SELECTOR_OF.setdefault(id(target), [])
  if selector not in _SELECTOR_OF[id(target)]:
    _SELECTOR_OF[id(target)].append(selector)
  # `Class.method.arg = v`: calls of that method on any instance receive the binding.
  parts = selector.split(".")
  if len(parts) >= 2 and inspect.isfunction(target):
    try:
      owner = _resolve_name(".".join(parts[:-1]), imports)
    except GinError:
      return
    if inspect.isclass(owner) and (id(owner), parts[-1]) not in _PATCHED_METHODS:
      orig = target
      _PATCHED_METHODS[(id(owner), parts[-1])] = orig

      @functools.wraps(orig)
      def method(self, *args, **kwargs):
        bound = _bindings_for(orig, selector, "")
        params = inspect.signature(orig).parameters
        positional = [p for p in list(params.values())[1:]
                      if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        passed = {p.name for p in positional[:len(args)]}
        for pname, (key, val) in bound.items():
          if pname not in kwargs and pname not in passed and pname in params:
            kwargs[pname] = _materialize(val)
            _OPERATIVE[key] = val
        return orig(self, *args, **kwargs)

      _SELECTOR_OF.setdefault(id(orig), []).append(selector)
      setattr(owner, parts[-1], method)


def parse_config_files_and_bindings(config_files: Optional[Sequence[str]],
                                    bindings: Optional[Sequence[str]],
                                    finalize_config: bool = True, skip_unknown: bool = False,
                                    print_includes_and_imports: bool = False) -> None:
  for f in config_files or []:
    parse_config_file(f, skip_unknown=skip_unknown)
  if bindings:
    parse_config(list(bindings), skip_unknown=skip_unknown)
  if finalize_config:
    finalize()


def finalize() -> None:
  global _FINALIZED
  _FINALIZED = True


def config_is_locked() -> bool:
  return _FINALIZED


# ----------------------------------------------------------------------------
# Dumping
# ----------------------------------------------------------------------------
def _dump(cfg: Dict[Tuple[str, str, str], Any]) -> str:
  macros = [(k, v) for k, v in cfg.items() if k[1] == "macro"]
  others = [(k, v) for k, v in cfg.items() if k[1] != "macro"]
  lines = []
  if macros:
    lines.append("# Macros:")
    lines.append("# " + "=" * 78)
    for (sc, _, p), v in macros:
      lines.append(f"{p} = {_format_value(v)}")
    lines.append("")
  groups: Dict[Tuple[str, str], List[Tuple[str, Any]]] = {}
  for (sc, sel, p), v in others:
    groups.setdefault((sc, sel), []).append((p, v))
  for (sc, sel), items in sorted(groups.items()):
    prefix = (sc + "/" if sc else "") + sel
    lines.append(f"# Parameters for {prefix}:")
    lines.append("# " + "=" * 78)
    for p, v in items:
      lines.append(f"{prefix}.{p} = {_format_value(v)}")
    lines.append("")
  return "\n".join(lines)


def config_str() -> str:
  return _dump(_CONFIG)


def operative_config_str() -> str:
  macros = {k: v for k, v in _CONFIG.items() if k[1] == "macro"}
  merged = dict(macros)
  merged.update(_OPERATIVE)
  return _dump(merged)


def markdown(string: str) -> str:
  """Formats a config string as Markdown (headers from the comment lines, code otherwise)."""
  out = []
  for line in string.split("\n"):
    if line.startswith("# ==="):
      continue
    if line.startswith("#"):
      out.append("#### " + line[1:].strip())
    elif line.strip():
      out.append("    " + line)
    else:
      out.append("")
  return "\n".join(out)
