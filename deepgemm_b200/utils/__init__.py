from . import math, layout
from .math import *  # noqa: F401,F403
from .layout import *  # noqa: F401,F403
