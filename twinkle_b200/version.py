__version__ = "0.1.0"
__release_datetime__ = "2099-12-31 23:59:59"  # placeholder of a source build, as in the reference's version.py
