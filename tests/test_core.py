

def test_nvtx_range_is_a_noop_without_cuda(monkeypatch):
    from optimus_dl_b200.core import profile

    monkeypatch.setattr(profile, "_NVTX", None)
    monkeypatch.setenv("OPTIMUS_NVTX", "1")
    with profile.nvtx_range("phase") as r:       # no CUDA device here: enabled flag resolves to False
        assert r.on == profile.nvtx_enabled()
    monkeypatch.setattr(profile, "_NVTX", None)
