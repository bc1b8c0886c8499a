"""Semantics of the gin-compatible configuration system on small configs: bindings and their
override order, macros, references (callable and evaluated), scopes, classes, method bindings,
REQUIRED, constants, queries, includes, literals, operative config."""
import os

import pytest

from t5x_b200 import gin
from tests import gin_test_targets as targets


@pytest.fixture(autouse=True)
def fresh_config():
  gin.clear_config(clear_constants=True)
  yield
  gin.clear_config(clear_constants=True)


HEADER = "from __gin__ import dynamic_registration\nfrom tests import gin_test_targets as tt\n"


def test_bindings_macros_and_override_order():
  gin.parse_config(HEADER + """
FACTOR = 3
tt.scaled.factor = %FACTOR
tt.scaled.offset = 1
tt.scaled.offset = 5      # the later binding wins
""")
  fn = gin.get_configurable(targets.scaled)
  assert fn(2) == 11
  assert fn(2, offset=0) == 6            # explicit arguments win over bindings
  assert gin.query_parameter("tt.scaled.offset") == 5
  assert gin.query_parameter("%FACTOR") == 3
  gin.bind_parameter("tt.scaled.factor", 10)
  assert fn(2) == 25
  with pytest.raises((gin.GinError, KeyError, ValueError)):
    gin.query_parameter("tt.scaled.missing")


def test_references_callable_and_evaluated():
  gin.parse_config(HEADER + """
tt.scaled.factor = 2
tt.make_pair.first = @tt.scaled        # the configured callable itself
tt.make_pair.second = @tt.Widget()     # a fresh result at every injection
tt.Widget.size = 7
""")
  first, second = gin.get_configurable(targets.make_pair)()
  assert first(4) == 8
  assert isinstance(second, targets.Widget) and second.size == 7
  _, again = gin.get_configurable(targets.make_pair)()
  assert again is not second


def test_scopes_select_bindings():
  gin.parse_config(HEADER + """
tt.Widget.size = 1
big/tt.Widget.size = 100
big/tt.Widget.name = "large"
tt.make_pair.first = @tt.Widget()
tt.make_pair.second = @big/tt.Widget()
""")
  small, big = gin.get_configurable(targets.make_pair)()
  assert (small.size, small.name) == (1, "w") and (big.size, big.name) == (100, "large")
  with gin.config_scope("big"):
    assert gin.get_configurable(targets.Widget)().size == 100
  assert gin.get_configurable(targets.Widget)().size == 1


def test_method_bindings_and_block_form():
  gin.parse_config(HEADER + """
tt.Widget:
  size = 4
  name = 'blocky'
tt.Widget.grow.by = 10
""")
  w = gin.get_configurable(targets.Widget)()
  assert (w.size, w.name) == (4, "blocky")
  assert w.grow() == 14 and w.grow(times=2) == 24 and w.grow(1) == 5


def test_required_constants_and_locking():
  gin.parse_config(HEADER + "tt.needs.value = %gin.REQUIRED\n")
  with pytest.raises((gin.GinError, TypeError, ValueError)):
    gin.get_configurable(targets.needs)()
  assert gin.get_configurable(targets.needs)(value=3) == 3
  gin.constant("my.CONST", 42)
  gin.parse_config(HEADER + "tt.needs.value = %my.CONST\n")
  assert gin.get_configurable(targets.needs)() == 42
  assert not gin.config_is_locked()
  gin.finalize()
  assert gin.config_is_locked()


def test_literals_and_multiline_values():
  assert gin.parse_value("[1, 2.5, 'a', None, True, (1, 2), {'k': [3]}]") == \
      [1, 2.5, "a", None, True, (1, 2), {"k": [3]}]
  assert gin.parse_value("'ab' 'cd'") == "abcd"
  assert gin.parse_value("(1,)") == (1,) and gin.parse_value("(1)") == 1
  assert gin.parse_value("-1e-3") == -1e-3 and gin.parse_value("{}") == {}
  gin.parse_config(HEADER + """
tt.make_pair.first = {
    'lengths': {'inputs': 512, 'targets': 114},   # a comment inside the value
    'names': ['a',
              'b'],
}
tt.make_pair.second = \\
    "continued"
""")
  first, second = gin.get_configurable(targets.make_pair)()
  assert first == {"lengths": {"inputs": 512, "targets": 114}, "names": ["a", "b"]}
  assert second == "continued"


def test_includes_search_paths_and_unknown_names(tmp_path):
  base = tmp_path / "base.gin"
  base.write_text(HEADER + "tt.scaled.factor = 2\ntt.scaled.offset = 1\n")
  child = tmp_path / "sub" / "child.gin"
  child.parent.mkdir()
  child.write_text("include 'base.gin'\ntt.scaled.offset = 9\n")
  gin.add_config_file_search_path(str(tmp_path))
  gin.parse_config_files_and_bindings([str(child)], ["tt.scaled.factor = 4"])
  assert gin.get_configurable(targets.scaled)(1) == 13       # 1 * 4 + 9
  with pytest.raises(gin.GinError):
    gin.parse_config(HEADER + "tt.no_such_function.arg = 1\n")
  gin.parse_config(HEADER + "tt.no_such_function.arg = 1\n", skip_unknown=True)
  with pytest.raises((gin.GinError, FileNotFoundError, OSError)):
    gin.parse_config_file(str(tmp_path / "missing.gin"))


def test_operative_config_lists_what_was_used():
  gin.parse_config(HEADER + """
LIMIT = 8
tt.scaled.factor = %LIMIT
tt.scaled.offset = 2
tt.Widget.size = 3
""")
  gin.get_configurable(targets.scaled)(1)
  full = gin.config_str()
  used = gin.operative_config_str()
  assert "tt.Widget.size = 3" in full and "tt.scaled.factor = %LIMIT" in full
  assert "tt.scaled.offset = 2" in used and "LIMIT = 8" in used
  assert "tt.Widget.size" not in used                      # never constructed
  md = gin.markdown(used)
  assert "#### Parameters for tt.scaled:" in md and "    tt.scaled.offset = 2" in md


def test_decorated_configurables_and_reference_module_aliases():
  @gin.configurable(module="unit")
  def rate(base=1.0, scale=1.0):
    return base * scale

  @gin.configurable
  class Counter:
    def __init__(self, start=0, step=1):
      self.start, self.step = start, step

  gin.parse_config("unit.rate.scale = 4.0\nCounter.step = 5\n")
  assert rate(base=2.0) == 8.0
  c = Counter(start=3)
  assert (c.start, c.step) == (3, 5)
  # names of the reference project resolve to this package
  gin.parse_config("from __gin__ import dynamic_registration\nfrom t5x import utils\n"
                   "utils.create_learning_rate_scheduler.warmup_steps = 7\n")
  from t5x_b200.utils import schedules
  assert gin.query_parameter("utils.create_learning_rate_scheduler.warmup_steps") == 7
  fn = gin.get_configurable(schedules.create_learning_rate_scheduler)(
      factors="constant * linear_warmup", base_learning_rate=1.0)
  assert fn(7) == pytest.approx(1.0) and fn(3) == pytest.approx(3 / 7)
