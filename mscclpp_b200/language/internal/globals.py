"""Import path kept for code written against the reference (`mscclpp.language.internal.globals`)."""
from .._context import get_program, set_program  # noqa: F401
