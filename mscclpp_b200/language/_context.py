"""The program that DSL calls currently append to (set by `with CollectiveProgram(...)`)."""
_current = None


def set_program(program) -> None:
    global _current
    _current = program


def get_program():
    if _current is None:
        raise RuntimeError("No Program in context")
    return _current
