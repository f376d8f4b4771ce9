"""What ``bench.py`` needs beside the engine: the shared measuring helpers, the arm that runs
the unmodified reference, and the offline install of the reference under ``baseline/_ref``
(which is not tracked)."""
