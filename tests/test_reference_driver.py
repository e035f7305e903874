"""The drop-in proof: the reference's own, unmodified benchmark / test driver (its
src/timing_layers.c with src/utils.c and src/tnns/data.c) linked against libtnns_b200.so in place of
the reference's objects (oracle/Makefile, target _ref/timing_layers_b200 -- the link line of
INTEGRATION.md).  On the CPU box: it builds and binds the drop-in symbols from this library.  On
the GPU box: its test mode runs the reference's 12 shapes through tnns_conv on the GPU and compares
every output with the reference's float convolution (src/timing_layers.c:142-165); exit code 0 means
all shapes passed."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
DRIVER = ROOT / "oracle" / "_ref" / "timing_layers_b200"


def test_reference_driver_links_against_the_library():
    from oracle import binding
    if binding.reference_checkout():
        binding.build()
    if not DRIVER.exists():
        pytest.skip("no reference checkout here and no prebuilt driver")
    dyn = subprocess.run(["readelf", "-d", str(DRIVER)], check=True, stdout=subprocess.PIPE, text=True).stdout
    assert "libtnns_b200.so" in dyn
    undefined = subprocess.run(["nm", "-D", "--undefined-only", str(DRIVER)], check=True, stdout=subprocess.PIPE, text=True).stdout
    assert " tnns_conv" in undefined, "the driver must take tnns_conv from the library"
    for own in ("mm_tnn", "t2r_p2_opt", "ternarize2row"):
        defined = subprocess.run(["nm", "--defined-only", str(DRIVER)], check=True, stdout=subprocess.PIPE, text=True).stdout
        assert f" {own}" not in defined, "none of the reference's hot-path objects may be linked in"


@pytest.mark.gpu
@pytest.mark.parametrize("net", ["tnn", "tbn", "btn", "bnn"])
def test_reference_driver_test_mode_passes_on_the_gpu(net, tmp_path):
    if not DRIVER.exists():
        pytest.skip("oracle/_ref/timing_layers_b200 was not built")
    (tmp_path / "out" / "measurements").mkdir(parents=True)
    r = subprocess.run([str(DRIVER), "cuda", net, "test"], cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-2000:]
    csvs = list((tmp_path / "out" / "measurements").glob("*.csv"))
    assert csvs, "the driver writes one measurement file per run"
    rows = csvs[0].read_text().strip().splitlines()
    assert len(rows) == 1 + 12, rows   # header + the 12 shapes of its correctness run
    keep = os.environ.get("TNNS_KEEP_MEASUREMENTS")
    if keep:
        shutil.copy(csvs[0], Path(keep) / f"reference_driver_{net}_test.csv")
