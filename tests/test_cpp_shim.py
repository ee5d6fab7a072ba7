"""The header-only C++ front (include/cphnsw/index/cp_hnsw_index.hpp): compiles and links against the
C-ABI library on any machine; its QA program (modelled on the reference's evaluation/qa_protocol.cpp)
runs on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "qa_protocol")


def compile_qa():
    lib_dir = os.path.join(ROOT, "sparse-text-kmeans_b200")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "qa_protocol.cpp"),
           "-L", lib_dir, "-lcphnsw_b200", "-Wl,-rpath," + lib_dir, "-o", EXE]
    subprocess.check_call(cmd)


def test_cpp_front_compiles_and_links(cp):
    compile_qa()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_cpp_qa_protocol(cp):
    compile_qa()
    out = subprocess.run([EXE], capture_output=True, text=True, timeout=600)
    print(out.stdout[-3000:], out.stderr[-2000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ALL PASS" in out.stdout


BIN_EXE = os.path.join(ROOT, "tests", "cpp", "binary_check")


def compile_binary():
    lib_dir = os.path.join(ROOT, "sparse-text-kmeans_b200")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([cxx, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "binary_check.cpp"),
                           "-L", lib_dir, "-lcphnsw_b200", "-Wl,-rpath," + lib_dir, "-o", BIN_EXE])


def test_binary_front_compiles_and_links(cp):
    compile_binary()
    assert os.path.exists(BIN_EXE)


@pytest.mark.gpu
def test_binary_front_runs(cp):
    compile_binary()
    out = subprocess.run([BIN_EXE], capture_output=True, text=True, timeout=600)
    print(out.stdout[-3000:], out.stderr[-2000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ALL PASS" in out.stdout


FRONT_EXE = os.path.join(ROOT, "tests", "cpp", "gpu_front_check")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def compile_gpu_fronts():
    lib_dir = os.path.join(ROOT, "sparse-text-kmeans_b200")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([cxx, "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA_HOME, "include"),
                           os.path.join(ROOT, "tests", "cpp", "gpu_front_check.cpp"), "-L", lib_dir, "-lcphnsw_b200",
                           "-L", os.path.join(CUDA_HOME, "lib64"), "-lcudart", "-Wl,-rpath," + lib_dir, "-o", FRONT_EXE])


def test_gpu_class_fronts_compile_and_link(cp):
    """include/cphnsw/cuda/gpu_encoder.cuh and gpu_knn_graph.cuh (GPUEncoder, GPUBruteForce, GPUKNNGraphBuilder)."""
    compile_gpu_fronts()
    assert os.path.exists(FRONT_EXE)


@pytest.mark.gpu
def test_gpu_class_fronts_run(cp):
    compile_gpu_fronts()
    out = subprocess.run([FRONT_EXE], capture_output=True, text=True, timeout=600)
    print(out.stdout[-3000:], out.stderr[-2000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ALL PASS" in out.stdout



OMP_EXE = os.path.join(ROOT, "tests", "cpp", "omp_search")


def compile_omp():
    lib_dir = os.path.join(ROOT, "sparse-text-kmeans_b200")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([cxx, "-std=c++17", "-O2", "-fopenmp", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "omp_search.cpp"), "-L", lib_dir, "-lcphnsw_b200",
                           "-Wl,-rpath," + lib_dir, "-o", OMP_EXE])


def test_omp_search_compiles_and_links(cp):
    """Searches from an OpenMP loop over one shared index (the loop shape of evaluation/eval_sift.cpp:380-387)."""
    compile_omp()
    assert os.path.exists(OMP_EXE)


@pytest.mark.gpu
def test_omp_search_runs(cp):
    compile_omp()
    out = subprocess.run([OMP_EXE], capture_output=True, text=True, timeout=600)
    print(out.stdout[-3000:], out.stderr[-2000:])
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "ALL PASS" in out.stdout
