"""The C++ host mirror (include/soklyn_b200.hpp) compiles warning-free against the C ABI and
passes its host-only checks: error variants and messages, schedulers, optimiser unpacking,
initialisers, seeds. No GPU needed; nothing here launches a kernel."""
import cpp_host


def test_cpp_host_mirror_builds_and_passes_host_checks():
    r = cpp_host.run("checks")
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("ok ")


def test_cpp_driver_rejects_bad_arguments():
    assert cpp_host.run().returncode == 2
    r = cpp_host.run("train", "/nonexistent/in", "/nonexistent/out")
    assert r.returncode == 3 and "cannot open" in r.stderr
