"""Keras data sets (bindings/python/old/flexflow/keras/datasets).  The legacy loaders download their files; these read the
same files from a local path and say which file they want when it is not there (nothing is fetched from the network)."""
from . import cifar10, mnist, reuters  # noqa: F401
