from ._context import get_program


def JSON() -> str:
    """The JSON plan of the program in context."""
    return get_program().to_json()
