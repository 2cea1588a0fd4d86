"""Launch rules as data: the tables and their resolver."""
from .resolve import LaunchDescriptor, Rules, RulesError, default_rules, set_default_rules  # noqa: F401
