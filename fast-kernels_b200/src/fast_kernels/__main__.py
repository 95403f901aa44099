from fast_kernels.cli.main import main

raise SystemExit(main())
