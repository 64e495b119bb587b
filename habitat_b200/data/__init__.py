"""Data files of the package (reference: analyzer/habitat/data/__init__.py:6-7)."""
import os

_HERE = os.path.abspath(os.path.dirname(__file__))


def path_to_data(data_file):
    return os.path.join(_HERE, data_file)
