from .merger import main

main()
