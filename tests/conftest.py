"""pytest configuration: registers the ``gpu`` marker.

No test carries it yet: no CUDA path exists in this repository, because the
reference project holds no MoE token-routing code to build one against.
"""


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (none defined yet)")
