"""Kept at the reference's path: ``from scripts.cli import parse_args``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hippolm_b200.cli import build_parser, parse_args, _flatten_optimizer_overrides, _load_yaml_with_extends  # noqa: E402,F401
