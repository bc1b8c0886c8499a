"""Plain callables for tests/test_gin_semantics.py to configure through dotted names."""


def scaled(x, factor=1, offset=0):
  return x * factor + offset


def make_pair(first=None, second=None):
  return (first, second)


class Widget:
  def __init__(self, size=1, name="w", part=None):
    self.size, self.name, self.part = size, name, part

  def grow(self, by=1, times=1):
    return self.size + by * times


def needs(value):
  return value
