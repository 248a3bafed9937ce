class Stmt:
    """Base class of the statements."""
