"""Alias of ``flashqla_b200.utils`` under the reference's module path."""

from flashqla_b200.utils import *  # noqa: F401,F403
from flashqla_b200.utils import __all__  # noqa: F401
