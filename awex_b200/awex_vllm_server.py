"""vLLM's OpenAI-compatible server with the weight-update routes and worker
methods of this framework registered:

    python -m awex_b200.awex_vllm_server <vllm serve arguments> [--awex-comm-backend nccl]

(`awex/awex_vllm_server.py:36-53` in the reference).  ``--awex-comm-backend``
and ``--awex-meta-server-addr`` are stripped from the argument list and exported
as ``AWEX_COMM_BACKEND`` / ``AWEX_META_SERVER_ADDR`` so that worker processes,
which vLLM spawns without our arguments, see them.
"""

from __future__ import annotations

import os
import sys
from typing import List, Optional, Tuple

_OWN_FLAGS = {"--awex-comm-backend": "AWEX_COMM_BACKEND", "--awex-meta-server-addr": "AWEX_META_SERVER_ADDR"}


def split_own_arguments(argv: List[str]) -> Tuple[List[str], dict]:
    """Separate this wrapper's flags (``--flag value`` or ``--flag=value``) from
    the arguments meant for vLLM."""
    rest, own, i = [], {}, 0
    while i < len(argv):
        token = argv[i]
        name, eq, value = token.partition("=")
        if name in _OWN_FLAGS:
            if not eq:
                if i + 1 >= len(argv):
                    raise SystemExit(f"{name} needs a value")
                value, i = argv[i + 1], i + 1
            own[_OWN_FLAGS[name]] = value
        else:
            rest.append(token)
        i += 1
    return rest, own


def _flexible_parser(description: str):
    try:
        from vllm.utils import FlexibleArgumentParser
    except ImportError:  # moved in newer releases
        from vllm.utils.argparse_utils import FlexibleArgumentParser
    return FlexibleArgumentParser(description=description)


def serve(argv: Optional[List[str]] = None) -> None:
    vllm_argv, exported = split_own_arguments(list(sys.argv[1:] if argv is None else argv))
    os.environ.update(exported)

    from awex_b200.vllm_plugin import register_awex_routes

    register_awex_routes()  # before vLLM builds its app and spawns workers

    import uvloop
    from vllm.entrypoints.openai import api_server, cli_args
    from vllm.entrypoints.utils import cli_env_setup

    cli_env_setup()
    parser = cli_args.make_arg_parser(_flexible_parser("vLLM OpenAI-compatible server with weight-update routes"))
    args = parser.parse_args(vllm_argv)
    cli_args.validate_parsed_serve_args(args)
    uvloop.run(api_server.run_server(args))


def main() -> None:
    serve()


if __name__ == "__main__":
    main()
