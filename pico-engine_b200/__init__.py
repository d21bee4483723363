"""Sources of the ``pico_engine`` package (see ``pico_engine/__init__.py`` at the repository
root, which puts this folder on its search path)."""
