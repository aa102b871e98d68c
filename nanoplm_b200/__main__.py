from nanoplm_b200.cli import main

if __name__ == "__main__":
    main()
