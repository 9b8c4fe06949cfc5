"""ctypes binding of the CPU golden model (test infrastructure only).

Only tests, the smoke check and the bench's CPU-baseline leg may import this
package; the shipped library never does.
"""
from .binding import Oracle, load_params, build  # noqa: F401
