"""``gelib.SO3type``: a dict l -> number of channels (python/src/gelib/SO3type.py:14-18 of GElib)."""


class SO3type(dict):

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
