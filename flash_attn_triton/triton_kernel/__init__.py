"""Module paths of the reference's kernel package, re-exported for drop-in imports."""
