class Body(tuple):
    """An immutable statement sequence; prints like the tuple it is."""

    def __new__(cls, statements=()):
        return super().__new__(cls, tuple(statements))

    def __getitem__(self, item):
        result = super().__getitem__(item)
        return Body(result) if isinstance(item, slice) else result
