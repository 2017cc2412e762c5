"""Reference-on-the-same-box runner (the reference package itself lives in ``baseline/_ref``, untracked)."""
