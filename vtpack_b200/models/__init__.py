from .dge import *  # noqa: F401,F403
