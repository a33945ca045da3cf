"""python -m seedpack_b200.refbind pack|unpack|test|list ... : the reference's command line with its kernels served by
libseedgrow.so (see seedpack_b200.refbind)."""
from . import main

main()
