      *> Calls the resonance bridge of libst_host from GnuCOBOL:
      *>   cobc -x RESONANCE.cbl -L../../spiraltorch_b200/_native -lst_host
      *> Five coefficients go in as COMP-1 (single-precision float); the summary comes back as a C string.
       IDENTIFICATION DIVISION.
       PROGRAM-ID. RESONANCE.
       DATA DIVISION.
       WORKING-STORAGE SECTION.
       01  WS-HANDLE          USAGE POINTER.
       01  WS-SUMMARY-PTR     USAGE POINTER.
       01  WS-STATUS          PIC S9(9) COMP-5.
       01  WS-LEN             PIC S9(9) COMP-5 VALUE 5.
       01  WS-CURVATURE       COMP-1 VALUE 0.42.
       01  WS-TEMPERATURE     COMP-1 VALUE 0.58.
       01  WS-COEFFICIENTS.
           05  WS-COEFF       COMP-1 OCCURS 5 TIMES.
       01  WS-SUMMARY         PIC X(255) BASED.
       01  WS-I               PIC 9(4) COMP-5.
       PROCEDURE DIVISION.
           MOVE 0.10  TO WS-COEFF(1)
           MOVE -0.30 TO WS-COEFF(2)
           MOVE 0.25  TO WS-COEFF(3)
           MOVE -0.40 TO WS-COEFF(4)
           MOVE 0.55  TO WS-COEFF(5)
           CALL "st_cobol_new_resonator" USING BY VALUE WS-CURVATURE
                                               BY VALUE WS-TEMPERATURE
                                         RETURNING WS-HANDLE
           IF WS-HANDLE = NULL
               DISPLAY "resonator could not be created"
               STOP RUN
           END-IF
           CALL "st_cobol_describe" USING BY VALUE WS-HANDLE
                                          BY REFERENCE WS-COEFFICIENTS
                                          BY VALUE WS-LEN
                                          BY REFERENCE WS-SUMMARY-PTR
                                    RETURNING WS-STATUS
           IF WS-STATUS = 0
               SET ADDRESS OF WS-SUMMARY TO WS-SUMMARY-PTR
               PERFORM VARYING WS-I FROM 1 BY 1
                       UNTIL WS-I > 255 OR WS-SUMMARY(WS-I:1) = X"00"
                   CONTINUE
               END-PERFORM
               DISPLAY WS-SUMMARY(1:WS-I - 1)
               CALL "st_cobol_free_string" USING BY VALUE WS-SUMMARY-PTR
           ELSE
               DISPLAY "describe failed with status " WS-STATUS
           END-IF
           CALL "st_cobol_free_resonator" USING BY VALUE WS-HANDLE
           STOP RUN.
