"""Command line: ``python -m tokenweave_b200 <command>`` (the counterpart of the reference's ``vllm`` CLI).

    serve   the OpenAI-compatible server (all flags of ``entrypoints/api_server.py``)
    build   compile the CUDA kernels into ``tokenweave_b200/_C.so``
    info    versions, devices and the kernels library in use
"""
import sys


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cmd = argv.pop(0) if argv else "--help"
    if cmd == "serve":
        from .entrypoints import api_server
        sys.argv = ["tokenweave_b200 serve"] + argv
        api_server.main()
        return 0
    if cmd == "build":
        from . import build
        print(build.build())
        return 0
    if cmd == "info":
        import torch
        from . import __version__
        from .ops import _native
        print(f"tokenweave_b200 {__version__}; torch {torch.__version__}; CUDA available: {torch.cuda.is_available()}")
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            print(f"  cuda:{i} {p.name}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.0f} GiB")
        print(f"  kernels: {_native._LIB_PATH} ({'present' if _native._LIB_PATH.exists() else 'not built'})")
        return 0
    print(__doc__)
    return 0 if cmd in ("-h", "--help", "help") else 2


if __name__ == "__main__":
    raise SystemExit(main())
