from . import teacache
