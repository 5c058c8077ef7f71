"""The MLIR module texts of the accelerated path live in the package (lapis_b200/modules.py); the tests
import them under their old name."""
from lapis_b200.modules import *  # noqa: F401,F403
