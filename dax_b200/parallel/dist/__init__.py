from . import coordinator, parallel_state
from .coordinator import *  # noqa: F401,F403
from .initialize import initialize, is_initialized
from .parallel_state import *  # noqa: F401,F403
