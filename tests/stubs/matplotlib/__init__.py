"""TEST-ONLY stand-in for matplotlib (absent from this image): just enough surface for the reference's
``run_nemotron_8b_decode_degradation.py`` to import it and "draw" its figure.  Nothing is rendered; saving
a figure writes a small text file that lists the plotted series."""

_backend = "agg"


def use(backend, **kwargs):
    global _backend
    _backend = str(backend).lower()


def get_backend():
    return _backend
