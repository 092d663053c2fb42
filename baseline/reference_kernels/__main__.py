import sys

from . import ReferenceUnavailable, build, fetch

if len(sys.argv) == 3 and sys.argv[1] == "fetch":
    print(fetch(sys.argv[2]))
elif len(sys.argv) == 2 and sys.argv[1] == "build":
    print(build())
else:
    print("usage: python -m baseline.reference_kernels fetch <reference checkout> | build", file=sys.stderr)
    sys.exit(2)
