"""Buildable-config (Fiddle-style) counterparts of the gin files: models, run configs, examples
(t5x/fiddle_configs/**)."""
