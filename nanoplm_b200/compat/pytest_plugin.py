"""`python -m pytest -p nanoplm_b200.compat.pytest_plugin ...`: serves the reference's import paths from this
package before any test module is imported."""
from nanoplm_b200 import compat

compat.install(force=True)
