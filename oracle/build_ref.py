"""Build the reference's own CPU implementation of the NN-evaluation path.

Test infrastructure only. Compiles the reference's sources *where they lie*
(nothing is copied into this repository) with g++ and links them with the
small driver programs in this directory:

  oracle/_ref/ref_eval   run a registered reference backend (blas / eigen) on a
                         weights file + position file and dump raw outputs
  oracle/_ref/mkpos      seeded legal playouts -> packed input planes
  oracle/_ref/mktd       V6 training-data records for seeded histories + the planes the reference reads back from them
  oracle/_ref/mkenc      seeded game histories + the reference encoder's planes for every input format / fill policy
  oracle/_ref/lc0_ref    the reference's own `lc0` binary (backendbench, check ...)

The recipe mirrors what the reference's meson build does (meson.build:60-124
proto generation, :128-206 source lists) without running meson: protobuf
headers come from the reference's scripts/compile_proto.py, the four
configure-time headers are written empty, and three include-path shims under
oracle/shim stand in for abseil and Eigen.  The `blas` flavour links the
OpenBLAS shared object that ships inside the opencv wheel when it exists;
otherwise only the plain-loop `eigen` flavour is registered.

usage: python oracle/build_ref.py [--reference /path/to/lc0] [--jobs N] [--extra-obj a.o ...]
"""
import argparse
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")

COMMON = """
src/chess/board.cc src/chess/gamestate.cc src/chess/position.cc src/chess/uciloop.cc
src/neural/backend.cc src/neural/batchsplit.cc src/neural/decoder.cc src/neural/encoder.cc
src/neural/factory.cc src/neural/loader.cc src/neural/register.cc src/neural/shared_params.cc
src/neural/wrapper.cc src/search/classic/node.cc src/syzygy/syzygy.cc src/trainingdata/reader.cc
src/trainingdata/trainingdata.cc src/trainingdata/writer.cc src/utils/commandline.cc
src/utils/configfile.cc src/utils/esc_codes.cc src/utils/files.cc src/utils/logging.cc
src/utils/optionsdict.cc src/utils/optionsparser.cc src/utils/random.cc src/utils/string.cc
src/version.cc
src/engine_loop.cc src/engine.cc src/neural/backends/network_check.cc
src/neural/backends/network_demux.cc src/neural/backends/network_mux.cc
src/neural/backends/network_random.cc src/neural/backends/network_record.cc
src/neural/backends/network_rr.cc src/neural/backends/network_trivial.cc src/neural/memcache.cc
src/neural/network_legacy.cc src/neural/onnx/adapters.cc src/neural/onnx/builder.cc
src/neural/onnx/converter.cc src/neural/xla/hlo_builder.cc src/neural/xla/onnx2hlo.cc
src/neural/xla/print_hlo.cc src/neural/xla/xla_tensor.cc src/search/classic/params.cc
src/search/classic/search.cc src/search/classic/stoppers/alphazero.cc
src/search/classic/stoppers/common.cc src/search/classic/stoppers/factory.cc
src/search/classic/stoppers/legacy.cc src/search/classic/stoppers/simple.cc
src/search/classic/stoppers/smooth.cc src/search/classic/stoppers/stoppers.cc
src/search/classic/stoppers/timemgr.cc src/search/classic/wrapper.cc src/search/register.cc
src/selfplay/game.cc src/selfplay/loop.cc src/selfplay/multigame.cc src/selfplay/tournament.cc
src/tools/backendbench.cc src/tools/benchmark.cc src/tools/describenet.cc src/tools/leela2onnx.cc
src/tools/onnx2leela.cc src/utils/histogram.cc src/utils/numa.cc src/utils/weights_adapter.cc
src/search/instamove/instamove.cc
src/utils/filesystem.posix.cc src/utils/trace.cc src/utils/protomessage.cc
src/neural/backends/blas/convolution1.cc src/neural/backends/blas/fully_connected_layer.cc
src/neural/backends/blas/se_unit.cc src/neural/backends/blas/network_blas.cc
src/neural/backends/blas/winograd_convolution3.cc
src/neural/backends/shared/activation.cc src/neural/backends/shared/winograd_filter.cc
""".split()


def find_openblas():
    import sysconfig
    site = sysconfig.get_paths()["purelib"]
    hits = sorted(glob.glob(os.path.join(site, "opencv_python_headless.libs", "libopenblasp-*.so")))
    return hits[0] if hits else None


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise SystemExit(1)


def build_cuda_reference(ref, obj, flags, common_objs, main_objs, link, jobs):
    """The reference's plain-CUDA backend as meson builds it with -Dplain_cuda=true -Dcudnn=false -Dcutlass=false
    (meson.build:539-581): layers.cc and network_cuda.cc with the host compiler, common_kernels.cu and
    fp16_kernels.cu with nvcc for sm_100, linked against cuBLAS."""
    cuda_home = "/usr/local/cuda"
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    cdir = os.path.join(ref, "src/neural/backends/cuda")
    inc = ["-I" + cdir, "-I" + os.path.join(cuda_home, "include")]
    objs = []
    for src in ("layers.cc", "network_cuda.cc"):
        o = os.path.join(obj, "cuda_" + src + ".o")
        if not os.path.exists(o):
            run(["g++"] + flags + inc + ["-c", os.path.join(cdir, src), "-o", o])
        objs.append(o)
    for src in ("common_kernels.cu", "fp16_kernels.cu"):
        o = os.path.join(obj, "cuda_" + src + ".o")
        if not os.path.exists(o):
            run([nvcc, "-arch=compute_100", "-code=sm_100", "-O3", "-std=c++20", "-Xcompiler", "-fPIC", "-w", "-DNO_PEXT"] +
                [f for f in flags if f.startswith("-I")] + inc + ["-c", os.path.join(cdir, src), "-o", o])
        objs.append(o)
    lib64 = os.path.join(cuda_home, "lib64")
    run(["g++", "-o", os.path.join(OUT, "ref_eval_cuda")] + common_objs + objs + main_objs + link +
        ["-L" + lib64, "-lcublas", "-lcudart", "-Wl,-rpath," + lib64])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "LC0_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")), help="root of the lc0 source tree")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--opt", default="-O2")
    ap.add_argument("--cuda", action="store_true",
                    help="also build oracle/_ref/ref_eval_cuda: the reference's own CUDA backend (cuBLAS GEMMs + its "
                         "SIMT kernels, no cuDNN / CUTLASS) for same-GPU comparison runs")
    ap.add_argument("--adapter", action="store_true",
                    help="also compile lc0_b200/adapter/network_b200.cc into lc0_ref/ref_eval")
    args = ap.parse_args()
    ref = args.reference
    if not os.path.isdir(ref):
        print("reference sources not found at", ref, "- nothing built")
        return 0
    gen = os.path.join(OUT, "gen")
    obj = os.path.join(OUT, "obj")
    os.makedirs(os.path.join(gen, "proto"), exist_ok=True)
    os.makedirs(obj, exist_ok=True)
    for p in ("net", "onnx", "hlo"):
        if not os.path.exists(os.path.join(gen, "proto", p + ".pb.h")):
            run([sys.executable, os.path.join(ref, "scripts/compile_proto.py"),
                 "--proto_path=" + ref, "--cpp_out=" + gen, os.path.join(ref, "proto", p + ".proto")])
    with open(os.path.join(gen, "build_id.h"), "w") as f:
        f.write('#define BUILD_IDENTIFIER "oracle-build"\n')
    for h in ("default_backend.h", "default_search.h", "trace_config.h"):
        open(os.path.join(gen, h), "a").close()

    blas = find_openblas()
    flags = ["-std=c++20", args.opt, "-DNO_PEXT", "-DNDEBUG", "-w",
             "-I" + os.path.join(HERE, "shim"), "-I" + os.path.join(ref, "src"), "-I" + gen,
             "-I" + os.path.join(ref, "third_party"), "-I" + ROOT]
    if blas:
        flags += ["-DUSE_BLAS", "-DUSE_OPENBLAS"]

    jobs = []
    for src in COMMON + ["src/main.cc"]:
        jobs.append((os.path.join(ref, src), os.path.join(obj, src.replace("/", "_") + ".o")))
    for src in ("ref_eval.cc", "mkpos.cc", "mkenc.cc", "mktd.cc"):
        jobs.append((os.path.join(HERE, src), os.path.join(obj, "oracle_" + src + ".o")))
    adapter_objs = []
    if args.adapter:
        a_src = os.path.join(ROOT, "lc0_b200", "adapter", "network_b200.cc")
        a_obj = os.path.join(obj, "adapter_network_b200.o")
        jobs.append((a_src, a_obj))
        adapter_objs.append(a_obj)

    def compile_one(job):
        src, o = job
        if os.path.exists(o) and os.path.getmtime(o) > os.path.getmtime(src):
            return
        run(["g++"] + flags + ["-c", src, "-o", o])

    with cf.ThreadPoolExecutor(args.jobs) as ex:
        list(ex.map(compile_one, jobs))

    common_objs = [o for (s, o) in jobs
                   if not s.endswith("main.cc") and not s.startswith(HERE) and o not in adapter_objs]
    link = ["-lz", "-lpthread", "-ldl"]
    if blas:
        d = os.path.dirname(blas)
        link += [blas, "-Wl,--disable-new-dtags", "-Wl,-rpath," + d, "-Wl,-rpath-link," + d]
    if adapter_objs:
        link += ["-Wl,-rpath,$ORIGIN/../../lc0_b200", "-L" + os.path.join(ROOT, "lc0_b200"), "-lb200nn"]

    def objof(name):
        return [o for (s, o) in jobs if s.endswith(name)]

    run(["g++", "-o", os.path.join(OUT, "ref_eval")] + common_objs + adapter_objs + objof("ref_eval.cc") + link)
    run(["g++", "-o", os.path.join(OUT, "mkpos")] + common_objs + objof("mkpos.cc") + link)
    run(["g++", "-o", os.path.join(OUT, "mkenc")] + common_objs + objof("mkenc.cc") + link)
    run(["g++", "-o", os.path.join(OUT, "mktd")] + common_objs + objof("mktd.cc") + link)
    run(["g++", "-o", os.path.join(OUT, "lc0_ref")] + common_objs + adapter_objs + objof("src/main.cc") + link)
    if args.cuda:
        build_cuda_reference(ref, obj, flags, common_objs, objof("ref_eval.cc"), link, args.jobs)
    print("built", OUT, "(blas flavour: %s)" % ("OpenBLAS " + blas if blas else "absent, eigen-shim only"))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
