from axlearn_b200.cli.main import main

if __name__ == "__main__":
    raise SystemExit(main())
