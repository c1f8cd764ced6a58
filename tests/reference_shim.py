"""pytest plugin (tests only): lets the reference's own test files import this
library under the reference's package name.

Loaded with ``-p reference_shim`` by ``test_reference_suite.py``.  It aliases
``swage_b200`` as ``swage`` and supplies the one name the reference's
segmented runner module exports that this library deliberately does not ship:
``cpu_oracle`` (``python/swage/_segmented_qualification.py:288-329``), taken
from the test-side oracle with the same calling convention.  Nothing in the
package depends on this file.
"""

import sys

import oracle
import swage_b200

swage_b200.install_as("swage")
sys.modules["swage._segmented_qualification"].cpu_oracle = oracle.cpu_oracle
