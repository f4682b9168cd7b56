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


def test_cpp_and_python_initialisers_draw_the_same_chacha8_values():
    """Both host mirrors restate ChaCha8Rng::seed_from_u64 + normal_dist / uniform_dist
    (src/util/function.rs:219-319): raw draws and the uniform initialisers agree bit for bit, the normal ones
    to the last bits of the platform's f32 log / cos."""
    import numpy as np
    import soklyn_b200 as sk
    from soklyn_b200.chacha import ChaCha8Rng
    cases = {"xavier_uniform": lambda s: sk.InitXavierUniformFunc(s, 0.5), "he_uniform": lambda s: sk.InitHeUniformFunc(s),
             "xavier_normal": lambda s: sk.InitXavierNormalFunc(s), "he_normal": lambda s: sk.InitHeNormalFunc(s, 2.0)}
    for kind, make in cases.items():
        seed, fi, fo, n = 20240607, 96, 40, 500
        r = cpp_host.run("draws", kind, str(seed), str(fi), str(fo), str(n))
        assert r.returncode == 0, r.stderr
        words = np.array([int(x, 16) for x in r.stdout.split()], dtype=np.uint32)
        assert np.array_equal(words[:8], ChaCha8Rng.seed_from_u64(seed).next_u32s(8))
        got = words[8:].view(np.float32)
        want = make(seed).init(fi, fo, n)
        if "uniform" in kind:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), kind
        else:
            assert np.allclose(got, want, rtol=2e-6, atol=1e-7), kind
