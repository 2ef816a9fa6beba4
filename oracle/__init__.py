"""CPU oracle for the SpMM path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline legs may import this
package; the product (cutespmm_ae_b200) never does.
"""
from .oracle import *  # noqa: F401,F403
